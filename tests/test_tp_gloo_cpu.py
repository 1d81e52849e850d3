"""Tensor-parallel host logic on CPU: two gloo ranks shard one decoder layer with eet_b200.tp's shard plan
(column-parallel QKV / gate / up, row-parallel O / down, quantize-then-shard scales), run the CPU oracle on
their shards, all-reduce the row-parallel partial outputs through eet_b200.tp.TensorParallel, and must
reproduce the unsharded oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from eet_b200 import tp as tp_mod
        from model_util import oracle_layers, random_hf_state_dict, tiny_config
        from oracle import ops
        tp = tp_mod.TensorParallel()
        assert (tp.rank, tp.size) == (rank, world)
        cfg = tiny_config(layers=1, hidden=256, heads=2, d_ff=192)   # 3 FFN tiles over 2 ranks: uneven split
        sd = random_hf_state_dict(cfg, seed=11)
        L = oracle_layers(sd, cfg)[0]
        h, D = cfg.hidden_size, 128
        h_lo, h_hi = tp_mod.head_range(cfg.num_attention_heads, rank, world)
        f_lo, f_hi = tp_mod.ff_range(cfg.intermediate_size, rank, world)
        a_lo, a_hi = h_lo * D, h_hi * D
        gen = torch.Generator().manual_seed(3)
        x = torch.randn(3, h, generator=gen).half()
        xn = ops.rmsnorm(x, L.ln1, 1e-6)
        # column-parallel fused QKV: this rank's columns of each of the Q, K, V blocks
        qkv_full = ops.gemm_w8a16(xn, L.qkv, L.qkv_s).view(3, 3, h)
        cols = torch.cat([torch.arange(a_lo, a_hi) + b * h for b in range(3)])
        qkv_mine = ops.gemm_w8a16(xn, L.qkv[:, cols], L.qkv_s[cols]).view(3, 3, a_hi - a_lo)
        assert torch.equal(qkv_mine, qkv_full[:, :, a_lo:a_hi])      # scales shard with the columns: bit-equal
        # row-parallel O projection on the rank's slice of a stand-in context, summed over ranks
        ctx = torch.randn(3, h, generator=gen).half()
        part = (ctx[:, a_lo:a_hi].float() @ ops.dequant(L.out[a_lo:a_hi], L.out_s)).contiguous()
        tp.all_reduce(part)
        want = ctx.float() @ ops.dequant(L.out, L.out_s)
        assert torch.allclose(part, want, rtol=1e-4, atol=1e-4)
        # FFN: column-parallel gate/up on uneven tile shards, row-parallel down, one all-reduce
        g = ops.gemm_w8a16(xn, L.gate[:, f_lo:f_hi], L.gate_s[f_lo:f_hi])
        u = ops.gemm_w8a16(xn, L.up[:, f_lo:f_hi], L.up_s[f_lo:f_hi])
        act = ops.gated_silu(g, u)
        part = (act.float() @ ops.dequant(L.down[f_lo:f_hi], L.down_s)).contiguous()
        tp.all_reduce(part)
        act_full = ops.gated_silu(ops.gemm_w8a16(xn, L.gate, L.gate_s), ops.gemm_w8a16(xn, L.up, L.up_s))
        want = act_full.float() @ ops.dequant(L.down, L.down_s)
        assert torch.allclose(part, want, rtol=1e-4, atol=1e-4)
        out_q.put((rank, "ok", (f_lo, f_hi)))
    except Exception as e:  # noqa: BLE001
        out_q.put((rank, f"{type(e).__name__}: {e}", None))
    finally:
        dist.destroy_process_group()


def test_sharded_oracle_equals_unsharded_over_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(r[1] for r in results) == ["ok", "ok"], results
    ranges = dict((r[0], r[2]) for r in results)
    assert ranges[0] == (0, 64) and ranges[1] == (64, 192)
