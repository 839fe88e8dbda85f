"""The installed vLLM driving this package as its platform plugin on a GPU: ``vllm.LLM`` on a small Llama-shaped
config with dummy weights runs through the plugin's platform class, attention backend, out-of-tree layers and the
tcgen05 GEMM; the test asserts that this package's kernels were launched.  Runs in a child process because vLLM
resolves its platform once per process."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, os, sys
sys.path.insert(0, os.environ["B200_ROOT"])
import torch
from vllm import LLM, SamplingParams
from vllm.platforms import current_platform
assert type(current_platform).__name__ == "B200Platform", type(current_platform)
from vllm_kunlun_b200.ops import _ext
llm = LLM(os.environ["B200_MODEL_DIR"], load_format="dummy", enforce_eager=True, skip_tokenizer_init=True,
          max_model_len=512, max_num_seqs=4, gpu_memory_utilization=0.3, block_size=64, dtype="bfloat16",
          enable_prefix_caching=False)
n0 = _ext.C().launch_count()
prompts = [{"prompt_token_ids": list(range(5, 5 + n))} for n in (40, 7)]
outs = llm.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True, detokenize=False))
n1 = _ext.C().launch_count()
toks = [list(o.outputs[0].token_ids) for o in outs]
from vllm.model_executor.custom_op import op_registry_oot
print("RESULT " + json.dumps({"launches": n1 - n0, "tokens": toks, "oot": sorted(op_registry_oot)}))
"""


def test_vllm_llm_runs_on_the_plugin():
    pytest.importorskip("vllm")
    d = tempfile.mkdtemp()
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 512, "intermediate_size": 1024,
           "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
           "vocab_size": 1024, "max_position_embeddings": 2048, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 1,
           "eos_token_id": 2}
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    from vllm_kunlun_b200._entry_points import write_egg_info
    write_egg_info(ROOT)
    env = dict(os.environ, B200_ROOT=ROOT, B200_MODEL_DIR=d, VLLM_ENABLE_V1_MULTIPROCESSING="0",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), VLLM_LOGGING_LEVEL="WARNING",
               TOKENIZERS_PARALLELISM="false")
    env.pop("VLLM_PLUGINS", None)
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=900)
    line = next((ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")), None)
    assert line is not None, f"child failed (rc {r.returncode})\n{r.stdout[-3000:]}\n{r.stderr[-6000:]}"
    res = json.loads(line[7:])
    assert res["launches"] > 0, "vLLM ran, but none of this package's kernels were launched"
    assert all(len(t) == 8 for t in res["tokens"]), res
    assert {"RMSNorm", "SiluAndMul", "RotaryEmbedding"} <= set(res["oot"])
