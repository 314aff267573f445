"""Worker for the multi-GPU data-parallel test: fused peer-memory step vs NCCL baseline, same data."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build(dev):
    from pmetal_b200.core.config import LoraConfig
    from pmetal_b200.lora import apply_lora
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    cfg = ModelArgs(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=2, num_key_value_heads=1, head_dim=128)
    m = DecoderLM(cfg).init_weights(0.05, 0)
    apply_lora(m, LoraConfig(r=16, alpha=32, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                             "up_proj", "down_proj"]), seed=1)
    m = m.to(dev)
    for n, p in m.named_parameters():
        if "lora_" not in n:
            p.data = p.data.to(torch.bfloat16)
    m.prepare_for_training()
    return m


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pmetal_b200.core.config import TrainingConfig
    from pmetal_b200.data.dataloader import synthetic_documents
    from pmetal_b200.data.packing import PackerConfig, SequencePacker, collate_packs
    from pmetal_b200.ops import native
    from pmetal_b200.parallel.dp import DistContext
    from pmetal_b200.parallel.fused_dp import FusedDataParallel
    from pmetal_b200.trainer.loop import TrainingLoop
    tc = TrainingConfig(learning_rate=1e-3, gradient_accumulation_steps=1, warmup_steps=0, lr_scheduler="constant",
                        max_grad_norm=0.5)
    docs = synthetic_documents(40, 20, 300, 2048, seed=10 + rank)
    packs = SequencePacker(PackerConfig(max_length=1024)).pack(docs)
    batches = [collate_packs(packs[i:i + 1], 1024).to(dev) for i in range(4)]
    results = {}
    for name, ctx in (("fused", FusedDataParallel(timeout_s=10.0)), ("nccl", DistContext())):
        model = build(dev)
        loop = TrainingLoop(model, tc, dist=ctx)
        for b in batches:
            loss, gn = loop.train_step(b)
        torch.cuda.synchronize()
        native.check_status()
        results[name] = (loop.opt.flat_p.clone(), float(loss))
        # all ranks must hold identical parameters after the step
        ref = loop.opt.flat_p.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, loop.opt.flat_p), f"{name}: parameters differ across ranks"
        if loop.opt.flat_shadow is not None:
            assert torch.allclose(loop.opt.flat_shadow.float(), loop.opt.flat_p, rtol=1e-2, atol=1e-3)
    pf, pn = results["fused"][0], results["nccl"][0]
    diff = (pf - pn).abs().max().item()
    mean_diff = (pf - pn).abs().mean().item()
    print(f"rank {rank}: fused vs nccl max param diff {diff:.3e} (loss fused {results['fused'][1]:.4f} "
          f"nccl {results['nccl'][1]:.4f})", flush=True)
    # LoRA weight gradients are accumulated with fp32 atomics (split-K), so two runs differ in the last bits and Adam's
    # normalised update can turn that into a full learning-rate step on elements whose gradient is ~0: bound the
    # mean tightly and the maximum by a few learning-rate steps
    assert mean_diff < 2e-5 and diff < 4e-3, (mean_diff, diff)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("DP_WORKER_OK", flush=True)
    sys.stdout.flush()
    from pmetal_b200.parallel.dp import shutdown_process_group
    shutdown_process_group()


if __name__ == "__main__":
    main()
