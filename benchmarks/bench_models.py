"""Model-shape benchmarks through the public API (device-timed, max over ranks, JSON per case):

  kimi_k2        4 stacked MoE blocks, H=7168, H'=2048 SwiGLU, epn=48, K=8, one shared expert,
                 S=4096 tokens/rank, forward+backward, routing skew swept over maxvio 0-3;
                 reports iteration time and peak memory.
  qwen3_30b_a3b  one MoE layer, H=2048, H'=768, epn=16 (E=128 at EP=8), K=8, S=8192 tokens/rank,
                 dispatch -> grouped GEMM -> combine forward and backward with reduce_grad,
                 maxvio in {0, 1, 2}.

    python benchmarks/bench_models.py --model kimi_k2 [--layers 4]      (or under torch.distributed.run)
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import calibrate_skew, barrier_sync, max_over_ranks  # noqa: E402
from moonep_b200.models.moe_block import MoEBlock, CONFIGS  # noqa: E402
from moonep_b200.ops import grouped_gemm as gg  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="kimi_k2", choices=["kimi_k2", "qwen3_30b_a3b", "deepseek_v3"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--maxvio", type=float, nargs="*", default=None)
    ap.add_argument("--private-slots", action="store_true",
                    help="every block gets its own Buffer and its own prefetch / reduce slots (default: the blocks "
                         "share one Buffer and one set of slots when there is more than one rank)")
    ap.add_argument("--optimizer", default="epilogue", choices=["epilogue", "after"],
                    help="experts' SGD in the epilogue of the weight-gradient GEMMs (default) or as kernels after the backward pass")
    ap.add_argument("--no-attention", action="store_true",
                    help="leave out the attention stand-in in front of every MoE layer (QKV projection, causal "
                         "scaled-dot-product attention over the rank's tokens as one sequence, output projection; "
                         "library kernels: it only gives the stack the compute a transformer block has between two MoE layers)")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl")
    cfg = CONFIGS[a.model]
    layers = a.layers or (4 if a.model == "kimi_k2" else 1)
    sweep = a.maxvio or ([0.0, 1.0, 2.0, 3.0] if a.model == "kimi_k2" else [0.0, 1.0, 2.0])
    shared_buf = shared_slots = None
    if world > 1 and layers > 1 and not a.private_slots:
        from moonep_b200 import Buffer
        from moonep_b200.pools import SharedSlots
        push = os.environ.get("MOONEP_PUSH_COMBINE", "1") != "0"
        shared_buf = Buffer(cfg.S, cfg.H, cfg.K, cfg.epn * world, world, num_sms=32, token_padding=cfg.token_padding,
                            push_combine=push)
        shared_slots = SharedSlots(cfg.epn, (cfg.H, cfg.Hp), (cfg.H, cfg.Hp), (cfg.Hp, cfg.H), with_grads=True)
    blocks = [MoEBlock(cfg, world, rank, num_sms=32, seed=l, buffer=shared_buf, shared_slots=shared_slots) for l in range(layers)]
    x0 = torch.randn(cfg.S, cfg.H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)).to(torch.bfloat16)
    lr = 1e-5
    if a.optimizer == "epilogue":
        for b in blocks:
            b.fuse_optimizer(lr, in_epilogue=True)
    attention = layers > 1 and not a.no_attention
    heads = max(1, cfg.H // 128)
    attn_w = []
    if attention:
        g = torch.Generator(device="cuda").manual_seed(1000 + rank)
        for _ in blocks:
            attn_w.append(((torch.randn(cfg.H, 3 * cfg.H, device="cuda", generator=g) * cfg.H ** -0.5).to(torch.bfloat16).requires_grad_(True),
                           (torch.randn(cfg.H, cfg.H, device="cuda", generator=g) * cfg.H ** -0.5).to(torch.bfloat16).requires_grad_(True)))

    def norm(h):
        return (h.float() * torch.rsqrt(h.float().pow(2).mean(dim=-1, keepdim=True) + 1e-6)).to(torch.bfloat16)

    def step():
        x = x0.detach().requires_grad_(True)
        h = x
        for i, b in enumerate(blocks):            # pre-norm residual stream
            if attention:
                wqkv, wo = attn_w[i]
                q, k, v = (norm(h) @ wqkv).view(cfg.S, 3, heads, cfg.H // heads).permute(1, 2, 0, 3).unsqueeze(1)
                o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
                h = h + o.squeeze(0).permute(1, 0, 2).reshape(cfg.S, cfg.H) @ wo
            h = h + b.forward(norm(h))
        loss = (h.float() ** 2).mean()
        loss.backward()
        for b in blocks:
            b.sgd_step(lr)
        for pair in attn_w:
            for w in pair:
                w.grad = None
        return loss.detach()

    for mv in sweep:
        real = 0.0
        for b in blocks:
            _, real = calibrate_skew(b, x0, mv, world)
        for _ in range(max(3, a.warmup)):
            step()
        torch.cuda.reset_peak_memory_stats()
        barrier_sync(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            loss = step()
        e1.record()
        barrier_sync(world)
        ms = max_over_ranks(e0.elapsed_time(e1) / a.steps, world)
        for b in blocks:
            b.buf.check()
        gg.check_status()
        if rank == 0:
            print(json.dumps({"model": cfg.name, "layers": layers, "n_gpus": world, "E": blocks[0].E,
                              "tokens_per_rank": cfg.S, "maxvio_target": mv, "maxvio": round(real, 3),
                              "iteration_ms": round(ms, 3), "tokens_per_s": round(cfg.S * world / ms * 1e3),
                              "peak_torch_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2),
                              "slots": "shared by all blocks" if shared_slots is not None else "one set per block",
                              "optimizer": a.optimizer, "attention_stand_in": attention,
                              "expert_and_comm_mem_gib": round((sum(b.pools.bytes_per_rank for b in blocks)
                                                                + (shared_slots.bytes_per_rank if shared_slots is not None else 0)
                                                                + sum(bf._heap.chunk_bytes for bf in {id(b.buf): b.buf for b in blocks}.values()))
                                                               / 2**30, 2),
                              "loss": float(loss)}), flush=True)
    for b in blocks:
        b.destroy()
    if shared_slots is not None:
        shared_slots.destroy()
    if shared_buf is not None:
        shared_buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
