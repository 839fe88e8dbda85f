"""``vllm-kunlun-b200 serve|bench|build`` command line."""
import sys


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: vllm-kunlun-b200 {serve,build,envs} ...")
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "serve":
        from .openai_server import main as serve
        return serve(rest)
    if cmd == "build":
        from ..build import build
        print(build(verbose="-v" in rest))
        return 0
    if cmd == "envs":
        from .. import envs
        for k, v in envs.describe().items():
            print(f"{k}={v}")
        return 0
    print(f"unknown command {cmd!r}")
    return 2


if __name__ == "__main__":
    sys.exit(main())
