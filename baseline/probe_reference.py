"""Can the unmodified reference plugin be imported on the vLLM that is installed here?

    python baseline/probe_reference.py [/path/to/reference]

The reference's offline ``pip install`` fails (its build backend ``hatchling`` is not in the wheelhouse), so this probe
takes a plain copy of the ``vllm_kunlun`` package, puts empty stand-ins for the four closed vendor wheels it imports at
module level (``kunlun_ops``, ``xspeedgate_ops``, ``cocopod``, ``xtorch_ops``) on ``sys.path`` and imports the modules
a dense model needs.  It prints one line per module and exits 0; nothing of this repository's engine or kernels is
involved.  ``bench.py --impl reference`` quotes the first failure as the reason for its ``unavailable`` line.
"""
import importlib
import os
import shutil
import sys
import tempfile
import traceback

MODULES = ["vllm_kunlun.platforms.kunlun", "vllm_kunlun.ops._custom_ops", "vllm_kunlun.ops",
           "vllm_kunlun.v1.attention.backends.kunlun_attn", "vllm_kunlun.v1.worker.utils",
           "vllm_kunlun.distributed.kunlun_communicator", "vllm_kunlun.ops.layernorm", "vllm_kunlun.models"]


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("B200_REFERENCE_DIR", "")   # a checkout of the reference
    here = os.path.dirname(os.path.abspath(__file__))
    installed = os.path.join(here, "_ref")
    work = tempfile.mkdtemp(prefix="refprobe_")
    if os.path.isdir(os.path.join(installed, "vllm_kunlun")):
        sys.path.insert(0, installed)
    elif os.path.isdir(os.path.join(ref, "vllm_kunlun")):
        shutil.copytree(os.path.join(ref, "vllm_kunlun"), os.path.join(work, "vllm_kunlun"))
        sys.path.insert(0, work)
    else:
        print("FAIL reference sources not found")
        return 0
    shim = os.path.join(work, "shim")
    os.makedirs(shim)
    for m in ("kunlun_ops", "xspeedgate_ops", "cocopod", "xtorch_ops"):
        open(os.path.join(shim, m + ".py"), "w").close()
    sys.path.insert(0, shim)
    import vllm
    print("vllm", vllm.__version__)
    import vllm_kunlun
    print("register ->", vllm_kunlun.register())
    for m in MODULES:
        try:
            importlib.import_module(m)
            print("OK  ", m)
        except Exception:
            last = traceback.format_exc().strip().splitlines()[-1]
            print("FAIL", m, "->", last)
    return 0


if __name__ == "__main__":
    sys.exit(main())
