"""CPU (gloo) worker: a continuous-batching engine on rank 0 over a model cut across the ranks; the other ranks hold no
scheduler and repeat rank 0's model calls from the step descriptors it publishes. The generated tokens equal those of an
engine over the whole model, with shared prompt prefixes and requests that join while others decode."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build():
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=8, model_type="qwen3_moe", num_experts=4, num_experts_per_tok=2,
                    moe_intermediate_size=32)
    m = DecoderLM(cfg).init_weights(0.2, 0).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def run_requests(engine, prompts):
    from pmetal_b200.models.sampling import SamplingParams
    from pmetal_b200.serve.engine import Request
    reqs = [engine.submit(Request(list(p), SamplingParams.greedy(6 + i))) for i, p in enumerate(prompts[:3])]
    for _ in range(3):
        engine.tick()
    reqs += [engine.submit(Request(list(p), SamplingParams.greedy(5))) for p in prompts[3:]]      # join mid-flight
    while not all(r.done.is_set() for r in reqs):
        engine.tick()
    return [r.output for r in reqs]


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    from pmetal_b200.parallel.tp_model import shard_for_serving
    from pmetal_b200.serve.engine import ContinuousBatchEngine
    from pmetal_b200.serve.replica import StepChannel, follow
    shared = list(range(3, 3 + 70))                 # longer than one cache block: the second request reuses its blocks
    prompts = [shared + [80, 81], [5, 9, 11], shared + [90], list(range(40, 60)), shared + [80, 81]]
    cut = build()
    shard_for_serving(cut)
    ch = cut.step_channel = StepChannel(StepChannel.control_group())
    if ch.leader:
        want = run_requests(ContinuousBatchEngine(build(), num_blocks=64, max_slots=4, prefill_chunk=48), prompts)
        eng = ContinuousBatchEngine(cut, num_blocks=64, max_slots=4, prefill_chunk=48)
        got = run_requests(eng, prompts)
        ch.stop()
        assert got == want, (got, want)
        assert eng.stats.prefix_hits >= 1 and ch.published > 10
    else:
        steps = follow(cut, cut.new_cache(64), ch)
        assert steps > 10
    dist.barrier()
    print("SERVE_REPLICA_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
