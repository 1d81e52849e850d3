"""Tensor-parallel model on 2, 4 and 8 GPUs (one process per GPU, NCCL for the plumbing) against the CPU oracle,
at the width the benchmark runs: two decoder layers of the LLaMA-7B architecture (hidden 4096, 32 heads, FFN
11008 - 86 strips of 128 channels, so the FFN shards are uneven at 4 and 8 ranks; int8 lm_head with its
vocabulary sharded over the ranks), batch 8, a 64-token prompt
and decode steps through the plain op calls (NCCL all-reduce), through the deferred-epilogue chain (the fused
exchange inside the RMSNorm head, with the cluster geometry and inbox addressing of the real hidden size) and
as a replayed CUDA graph.  Rank 0 compares its logits with the oracle; all ranks must hold bit-identical
logits, because every rank adds the partial rows in rank order.  A small uneven case (3 FFN tiles over 2
ranks) runs as well.  Skipped for world sizes the box does not have.

Tolerance: |err| <= 2e-2 + 2e-2 * |ref| on fp32 logits (as in the single-GPU model tests); in the NCCL path the
partial sums are rounded to fp16 before they are added, which stays inside it."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q, small, batch=8):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import torch.distributed as dist
        from eet_b200 import EET, _lib, modeling, tp as tp_mod
        from model_util import OracleLM, random_hf_state_dict, tiny_config
        tp = tp_mod.init_from_env("nccl")
        dev = torch.device("cuda", rank)
        if small:
            cfg = tiny_config(layers=2, hidden=512, heads=4, d_ff=192)      # 3 FFN tiles over 2 ranks: uneven
            B, S, NEW, T = 2, 6, 4, 16
        else:
            cfg = tiny_config(layers=2, hidden=4096, heads=32, d_ff=11008, vocab=1024)
            B, S, NEW, T = batch, 64, 4, 80
        sd = random_hf_state_dict(cfg, seed=9)
        eet_dict = modeling.convert_llama_weights({k: v.to(dev) for k, v in sd.items()}, torch.int8)
        gen = torch.Generator().manual_seed(1)
        ids = torch.randint(0, cfg.vocab_size, (B, S + NEW), generator=gen)
        # the full-width case also quantizes the lm_head and shards its 1024-entry vocabulary (16 tiles: even over
        # 2, 4, 8 ranks); the small case keeps the reference's replicated fp16 head
        head_int8 = not small
        model = modeling.EETLlamaForCausalLM.from_eet(eet_dict, cfg, B, S, T, torch.int8, device_id=rank, tp=tp,
                                                      lm_head_int8=head_int8)
        del eet_dict
        outs = [model(ids[:, :S].to(dev), first_pass=True).logits.float().cpu()]
        for i, t in enumerate(range(S, S + NEW)):
            step_ids = ids[:, t:t + 1].to(dev)
            if i < 2:     # plain op calls: NCCL all-reduce + separate residual kernel
                outs.append(model(step_ids, first_pass=False).logits.float().cpu())
            else:         # the chain generation uses: fused exchange in the next block's RMSNorm head
                outs.append(model.decode_logits(step_ids).float().cpu())
        toks = model.generate(ids[:, :S].to(dev), NEW + 2).cpu()
        model.use_cuda_graph = True
        toks_g = model.generate(ids[:, :S].to(dev), NEW + 2).cpu()
        torch.cuda.synchronize()
        assert _lib.device_status() == 0, "a bounded wait ran out"
        # every rank holds the same logits, bit for bit
        mine = torch.cat([o.reshape(-1) for o in outs[1:]]).to(dev)
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        assert all(torch.equal(e, mine) for e in everyone), "ranks disagree on the decode logits"
        outcome = [None]
        if rank == 0:
            try:
                lm = OracleLM(sd, cfg, max_len=T, batch=B, lm_head_int8=head_int8)
                want = [lm(ids[:, :S], True)] + [lm(ids[:, t:t + 1], False) for t in range(S, S + NEW)]
                for i, (a, b) in enumerate(zip(outs, want)):
                    err = (a - b).abs()
                    assert bool((err <= 2e-2 + 2e-2 * b.abs()).all()), f"output {i}: max err {float(err.max())}"
                # greedy tokens (eager, then as a replayed CUDA graph) against the oracle's wherever its top-2
                # margin is clear of the tolerance; the oracle follows the library's tokens (same history)
                for name, seq in (("eager", toks), ("graph", toks_g)):
                    lm2 = OracleLM(sd, cfg, max_len=T, batch=B, lm_head_int8=head_int8)
                    logits = lm2(ids[:, :S], True)[:, -1]
                    for t in range(NEW + 2):
                        top2 = logits.topk(2, -1).values
                        clear = (top2[:, 0] - top2[:, 1]) > 4e-2 + 4e-2 * top2[:, 0].abs()
                        tok = seq[:, S + t]
                        assert torch.equal(tok[clear], logits.argmax(-1)[clear]), f"{name}: generated token {t}"
                        logits = lm2(tok.view(B, 1), False)[:, -1]
            except AssertionError as e:
                outcome[0] = f"rank 0 against the oracle: {e}"
        # everybody learns the outcome, so that no rank is left waiting for one that has already given up
        dist.broadcast_object_list(outcome, src=0)
        assert outcome[0] is None, outcome[0]
        dist.barrier()
        q.put((rank, "ok"))
        # graphs that captured NCCL kernels must go before the communicator does
        model.end_graph()
        del model
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()[-2000:]))


def _run(world, small, batch=8):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 1000) + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, small, batch)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            # a rank that failed leaves the others waiting in a collective: do not wait long for them
            results.append(q.get(timeout=600 if all(r[1] == "ok" for r in results) else 20))
    except Exception:  # noqa: BLE001  (queue.Empty)
        results.append((-1, "no answer from the remaining ranks"))
    finally:
        for p in procs:
            p.join(timeout=30 if all(r[1] == "ok" for r in results) else 2)
            if p.is_alive():     # a stuck teardown must not outlive the test
                p.kill()
    assert sorted(r[1] for r in results) == ["ok"] * world, results


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_tensor_parallel_small_uneven_shards():
    _run(2, small=True)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_llama7b_width_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, small=False)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_fused_exchange_above_16_rows():
    """Batch 32 (the Baichuan-13B decode batch): the fused exchange with more than 16 rows per inbox, fed by the
    stream-K tensor-core GEMM instead of the skinny one, and the sharded lm_head's greedy kernel with 32 rows."""
    _run(2, small=False, batch=32)
