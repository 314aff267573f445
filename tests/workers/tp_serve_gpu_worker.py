"""Worker for the multi-GPU serving test: a model cut into tensor-parallel attention and expert-parallel feed-forward
slices against the whole model on one GPU (logits of a prefill and of decode / verification steps), with the NCCL sum
and with the one-kernel peer all-reduce; then the peer all-reduce alone over many calls and sizes."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build(dev):
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                    num_key_value_heads=2, head_dim=128, model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2,
                    moe_intermediate_size=256)
    m = DecoderLM(cfg).init_weights(0.05, 0).to(dev).to(torch.bfloat16).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pmetal_b200.models.generation import Generator
    from pmetal_b200.ops import native
    from pmetal_b200.parallel.tp_model import AllReduce, PeerAllReduce, shard_for_serving
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (70, 200, 33, 129, 5, 64, 257, 90, 17, 140, 31, 128, 99, 7, 180, 55)]
    whole = build(dev)
    ref_gen = Generator(whole, num_blocks=64, cuda_graphs=False)
    seqs = [ref_gen.new_seq() for _ in prompts]
    ref_pre = ref_gen.prefill(seqs, prompts).float()
    nxt = ref_pre.argmax(-1)
    ref_dec = ref_gen.decode_step(seqs, nxt).float()
    peer = PeerAllReduce(None, max_elems=1 << 16, timeout_s=5.0)
    for name, red in (("nccl", AllReduce(None)), ("peer", peer)):
        cut = build(dev)
        shard_for_serving(cut, None, red)
        gen = Generator(cut, num_blocks=64, cuda_graphs=False)
        s2 = [gen.new_seq() for _ in prompts]
        pre = gen.prefill(s2, prompts).float()
        dec = gen.decode_step(s2, nxt).float()
        torch.cuda.synchronize()
        native.check_status()
        for what, a, b in (("prefill", pre, ref_pre), ("decode", dec, ref_dec)):
            # bf16 partial sums arrive in another order than in the whole model, and a router near a tie may then pick
            # another expert for a token: the check is on the relative error of the whole logit matrix
            rows = ((a - b).norm(dim=-1) / b.norm(dim=-1)).tolist()
            if rank == 0:
                print(f"{name} {what}: relative error per row " + " ".join(f"{e:.3f}" for e in rows), flush=True)
            srt = sorted(rows)
            assert srt[len(srt) // 2] < 0.03 and srt[(3 * len(srt)) // 4 - 1] < 0.06, f"{name} {what}: {rows}"
        # every rank holds the same logits
        got = [torch.empty_like(dec) for _ in range(world)]
        dist.all_gather(got, dec)
        assert all(torch.equal(got[0], x) for x in got), f"{name}: ranks differ"
    # one mixture-of-experts block on identical inputs: whole against the sum of the slices, few and many tokens
    blk_w, blk_c = whole.layers[1].mlp, cut.layers[1].mlp
    for T in (4, 300, 5000):
        x = (0.5 * torch.randn(T, 512, device=dev, generator=torch.Generator(device=dev).manual_seed(T))).bfloat16()
        dist.broadcast(x, 0)
        with torch.no_grad():
            a, b = blk_c(x, x).float(), blk_w(x, x).float()
        rows = ((a - b).norm(dim=-1) / b.norm(dim=-1))
        bad = (rows > 0.02).float().mean().item()
        if rank == 0:
            print(f"block T={T}: median {rows.median().item():.4f} max {rows.max().item():.3f} rows over 2 %: {bad:.3f}",
                  flush=True)
        assert rows.median().item() < 0.01 and bad < 0.05, f"block T={T}"
    # continuous batching over the cut model, decode steps replayed from graphs: every rank running its own scheduler in
    # lock-step against rank 0 scheduling alone while the others repeat its steps from the published descriptors
    from pmetal_b200.models.sampling import SamplingParams
    from pmetal_b200.serve.engine import ContinuousBatchEngine, Request
    from pmetal_b200.serve.replica import StepChannel, follow

    def run_requests(engine):
        reqs = [engine.submit(Request(list(p), SamplingParams.greedy(8 + i))) for i, p in enumerate(prompts[:5])]
        for _ in range(4):
            engine.tick()
        reqs += [engine.submit(Request(list(p), SamplingParams.greedy(6))) for p in prompts[5:9]]
        while not all(r.done.is_set() for r in reqs):
            engine.tick()
        return [r.output for r in reqs]
    want = run_requests(ContinuousBatchEngine(cut, num_blocks=128, max_slots=8))
    ch = cut.step_channel = StepChannel(StepChannel.control_group())
    if ch.leader:
        got = run_requests(ContinuousBatchEngine(cut, num_blocks=128, max_slots=8))
        ch.stop()
        assert got == want, (got, want)
        print(f"engine with follower ranks: {len(got)} requests, {ch.published} step descriptors", flush=True)
    else:
        assert follow(cut, cut.new_cache(128), ch) > 10
    cut.step_channel = None
    torch.cuda.synchronize()
    native.check_status()
    # the peer all-reduce by itself: sizes up to the slot size, many calls back to back (both buffer halves, epochs)
    for it in range(12):
        n = [8, 4096, 1 << 16, 520 * 8][it % 4]
        x = (torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(100 * it + rank))).bfloat16()
        want = x.float().clone()
        dist.all_reduce(want)
        peer(x)
        assert (x.float() - want).abs().max().item() <= 0.02 * want.abs().max().item() + 1e-2, f"peer all-reduce call {it}"
    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    if rank == 0:
        print("TP_SERVE_GPU_WORKER_OK", flush=True)
    sys.stdout.flush()
    del peer
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    main()
