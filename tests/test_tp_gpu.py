"""Tensor-parallel model on two GPUs (NCCL): the sharded model must reproduce the single-GPU model's logits
(prefill and decode, eager and CUDA graph).  Skipped on a box with one GPU."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        import torch.distributed as dist
        from eet_b200 import modeling, tp as tp_mod
        from model_util import random_hf_state_dict, tiny_config
        tp = tp_mod.init_from_env("nccl")
        cfg = tiny_config(layers=2, hidden=512, heads=4, d_ff=192)      # 3 FFN tiles over 2 ranks: uneven
        sd = random_hf_state_dict(cfg, seed=9)
        eet_dict = modeling.convert_llama_weights({k: v.clone() for k, v in sd.items()}, torch.int8)
        B, S, T = 2, 6, 16
        gen = torch.Generator().manual_seed(1)
        ids = torch.randint(0, cfg.vocab_size, (B, S + 3), generator=gen)
        dev = torch.device("cuda", rank)
        sharded = modeling.EETLlamaForCausalLM.from_eet(eet_dict, cfg, B, 8, T, torch.int8, device_id=rank, tp=tp)
        outs = [sharded(ids[:, :S].to(dev), first_pass=True).logits.float().cpu()]
        for t in range(S, S + 3):
            outs.append(sharded(ids[:, t:t + 1].to(dev), first_pass=False).logits.float().cpu())
        toks = sharded.generate(ids[:, :S].to(dev), 4).cpu()
        sharded.use_cuda_graph = True
        toks_g = sharded.generate(ids[:, :S].to(dev), 4).cpu()
        if rank == 0:
            single = modeling.EETLlamaForCausalLM.from_eet(eet_dict, cfg, B, 8, T, torch.int8, device_id=0)
            ref = [single(ids[:, :S].to(dev), first_pass=True).logits.float().cpu()]
            for t in range(S, S + 3):
                ref.append(single(ids[:, t:t + 1].to(dev), first_pass=False).logits.float().cpu())
            for a, b in zip(outs, ref):
                # partial sums are rounded to fp16 before the all-reduce: a few fp16 ulps on O(1) activations
                assert torch.allclose(a, b, atol=3e-2, rtol=3e-2), float((a - b).abs().max())
            assert torch.equal(toks, toks_g)
        dist.barrier()
        q.put((rank, "ok"))
        # graphs that captured NCCL kernels must go before the communicator does
        sharded.end_graph()
        del sharded
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()[-1500:]))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_tensor_parallel_matches_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():     # a stuck teardown must not outlive the test
            p.kill()
    assert sorted(r[1] for r in results) == ["ok", "ok"], results
