"""CPU (gloo) worker: causal ring attention against full attention, pipeline inference against the single-process
model, and a 1F1B training schedule against plain backpropagation."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    from pmetal_b200.parallel import cp, pipeline, plans
    torch.manual_seed(0)
    # ---- ring attention
    T, hq, hkv, d = 8 * world, 4, 2, 16
    q, k, v = torch.randn(T, hq, d), torch.randn(T, hkv, d), torch.randn(T, hkv, d)
    out, lse = cp.ring_attention_p2p(cp.split_sequence(q, rank, world), cp.split_sequence(k, rank, world),
                                     cp.split_sequence(v, rank, world))
    kk, vv = k.repeat_interleave(2, 1).permute(1, 0, 2), v.repeat_interleave(2, 1).permute(1, 0, 2)
    s = torch.einsum("thd,hsd->hts", q, kk) / d ** 0.5
    s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
    ref = torch.einsum("hts,hsd->thd", s.softmax(-1), vv)
    mine = cp.split_sequence(ref, rank, world)
    assert torch.allclose(out, mine, atol=1e-5), (out - mine).abs().max()
    assert torch.allclose(lse, cp.split_sequence(torch.logsumexp(s, -1), rank, world, dim=1), atol=1e-5)
    full = cp.gather_sequence(out)
    assert torch.allclose(full, ref, atol=1e-5)
    # ---- pipeline inference
    cfg = ModelArgs(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=16)
    model = DecoderLM(cfg).init_weights(0.1, 0).eval()
    ranges = plans.assign_layers_proportional(4, [1.0] * world)
    a, b = ranges[rank]
    stage = pipeline.PipelineStage(model, a, b, rank, world)
    ids = torch.arange(1, 12)
    tok = stage.step(ids if rank == 0 else None, nonce=7)
    if rank == 0:
        with torch.no_grad():
            want = int(model(ids)[-1].argmax())
        assert tok == want, (tok, want)
    # ---- 1F1B training on a chain of linear stages
    torch.manual_seed(1)
    M = 4
    ws = [torch.randn(8, 8) * 0.3 for _ in range(world)]
    xs = {m: torch.randn(3, 8) for m in range(M)}
    w = ws[rank].clone().requires_grad_(True)
    sched = plans.schedule_1f1b(world, M, rank)
    losses = pipeline.run_schedule(sched, lambda x: torch.tanh(x @ w), xs, rank, world,
                                   loss_fn=lambda y, m: (y ** 2).mean(), activation_like=torch.empty(3, 8))
    ref_ws = [t.clone().requires_grad_(True) for t in ws]
    tot = 0
    for m in range(M):
        h = xs[m]
        for t in ref_ws:
            h = torch.tanh(h @ t)
        tot = tot + (h ** 2).mean()
    tot.backward()
    assert torch.allclose(w.grad, ref_ws[rank].grad, atol=1e-6), (w.grad - ref_ws[rank].grad).abs().max()
    if rank == world - 1:
        assert abs(sum(losses) - float(tot.detach())) < 1e-5
    dist.barrier()
    if rank == 0:
        print("CP_PP_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
