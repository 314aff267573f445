"""Start the OpenAI-compatible server on a model and stream one chat completion from it.

    python examples/serve_client.py --model random:tiny-qwen3 --device cpu

The server is the same one ``python -m pmetal_b200.cli.main serve`` runs; here it lives in a child process so that the
example is self-contained. Any OpenAI client can talk to it on the printed address."""
import argparse
import json
import os
import signal
import subprocess
import sys
import time
import urllib.request


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:tiny-qwen3")
    ap.add_argument("--port", type=int, default=18555)
    ap.add_argument("--device", default=None)
    ap.add_argument("--prompt", default="Say hello.")
    a = ap.parse_args()
    cmd = [sys.executable, "-m", "pmetal_b200.cli.main", "serve", "-m", a.model, "--port", str(a.port), "--kv-blocks", "256",
           "--max-slots", "4"] + (["--device", a.device] if a.device else [])
    server = subprocess.Popen(cmd, start_new_session=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    base = f"http://127.0.0.1:{a.port}"
    try:
        for _ in range(240):
            try:
                urllib.request.urlopen(base + "/health", timeout=1).read()
                break
            except Exception:
                if server.poll() is not None:
                    raise SystemExit("the server exited; run the serve command by hand to see why")
                time.sleep(0.5)
        body = {"messages": [{"role": "user", "content": a.prompt}], "max_tokens": 16, "temperature": 0, "stream": True}
        req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        pieces = []
        with urllib.request.urlopen(req, timeout=120) as resp:
            for raw in resp:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                delta = json.loads(line[6:])["choices"][0]["delta"]
                pieces.append(delta.get("content") or "")
        print(json.dumps({"address": base, "text": "".join(pieces)}))
    finally:
        os.killpg(server.pid, signal.SIGINT)
        try:
            server.wait(30)
        except subprocess.TimeoutExpired:
            os.killpg(server.pid, signal.SIGKILL)


if __name__ == "__main__":
    main()
