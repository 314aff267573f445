"""LoRA fine-tuning through the Python API, then generation with the adapter.

    python examples/finetune_lora.py --model random:tiny-qwen3 --steps 5 --device cpu
    python examples/finetune_lora.py --model /path/to/Qwen3-0.6B --data my.jsonl --steps 200

``--data`` is a JSONL file with a ``text`` column (or chat ``messages``); without it a few lines are written to a temporary
file so that the script runs as it is."""
import argparse
import json
import os
import tempfile

import pmetal_b200 as pm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:tiny-qwen3")
    ap.add_argument("--data")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--out", default=None)
    ap.add_argument("--device", default=None)
    a = ap.parse_args()
    work = tempfile.mkdtemp(prefix="pmetal-example-")
    data = a.data
    if not data:
        data = os.path.join(work, "train.jsonl")
        with open(data, "w", encoding="utf-8") as fh:
            for i in range(32):
                fh.write(json.dumps({"text": f"Question {i}: what is {i} plus {i}? Answer: {2 * i}."}) + "\n")
    out = a.out or os.path.join(work, "adapter")
    extra = {"device": a.device, "dtype": "float32"} if a.device == "cpu" else {}
    summary = pm.finetune(a.model, data, output=out, lora_r=8, lora_alpha=16.0, learning_rate=2e-4, max_steps=a.steps,
                          batch_size=2, **extra)
    print(json.dumps({"steps": summary["steps"], "final_loss": round(summary["final_loss"], 4), "adapter": summary["adapter"]}))
    model = pm.Model.load(a.model, lora=out, device=a.device)
    print(model.generate("Question 3: what is 3 plus 3? Answer:", max_tokens=8, temperature=0))


if __name__ == "__main__":
    main()
