"""Tensor parallelism for the int8 LLaMA / Baichuan path: Megatron-style sharding with one all-reduce
per row-parallel projection.  The reference is single-GPU (it has no communication layer at all); this
module is an addition on top of its operator API.

One process per GPU.  Column-parallel: fused QKV (by heads), gate and up (by d_ff).  Row-parallel: the
attention output projection and the FFN down projection; their partial outputs are summed over the group
and the residual is added after the sum.  RMSNorm weights, embedding and lm_head are replicated.
"""
import os

import torch
import torch.distributed as dist


class TensorParallel:
    """Handle passed to MetaDesc(tp=...).  Wraps a torch.distributed process group (NCCL on GPUs, gloo in
    CPU tests)."""

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def peer_buffers(self, hidden, device):
        """Creates (once) the peer-addressable buffers of the fused all-reduce for this hidden size."""
        if getattr(self, "_peer", None) is None or self._peer.hidden != hidden:
            self._peer = PeerBuffers(self, hidden, device)
        return self._peer

    def reset_peer_buffers(self):
        """Collective: every rank clears its partial sums, inbox and epoch counters, then all meet at a barrier.
        Needed after a rank reported device status 4 (a peer's sums never arrived): the epochs of the ranks may
        have diverged."""
        if getattr(self, "_peer", None) is not None:
            self._peer.clear_local()
            torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def all_reduce(self, tensor):
        """In-place sum over the group on the current stream."""
        if self.size > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor


class PeerBuffers:
    """What the fused tensor-parallel exchanges need on every rank: two local fp32 partial-sum buffers
    [rows][hidden] (attention-output / FFN-down projections alternate between them), an inbox
    [2][8 source ranks][rows][hidden / 8][3] of 16-byte packets {value, value, value, epoch} that the OTHER
    ranks write into over NVLink (eet_rmsnorm_finalize_tp), and behind it a small inbox [2][8][rows] of
    {logit, index, epoch} packets for the greedy token choice over a sharded vocabulary (eet_lm_head_argmax).
    The inboxes are shared through CUDA IPC handles exchanged over the process group.  Lets the decode path
    replace `NCCL all-reduce -> RMSNorm` by one kernel."""

    ROWS = 64

    def __init__(self, tp, hidden, device):
        import ctypes
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        from torch.multiprocessing.reductions import reduce_tensor
        self.tp, self.hidden = tp, hidden
        n = self.ROWS * hidden
        self.local_sums = torch.zeros(2 * n, dtype=torch.float32, device=device)
        sum_words = 2 * 8 * self.ROWS * (hidden // 8) * 3 * 4        # 16-byte packets, 3 per 8 values
        argmax_words = 2 * 8 * self.ROWS * 4                         # one 16-byte packet per (half, rank, row)
        self.local_inbox = torch.zeros(sum_words + argmax_words, dtype=torch.int32, device=device)
        self.epochs = torch.zeros(2 * self.ROWS, dtype=torch.int32, device=device)
        self.argmax_epochs = torch.zeros(self.ROWS, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        everyone = [None] * tp.size
        dist.all_gather_object(everyone, (reduce_tensor(self.local_inbox), device.index), group=tp.group)

        def open_on_my_device(reduced, exporter_index):
            # The handle is opened with THIS rank's device current, so the peer's memory is mapped into this
            # device's address space (the driver enables peer access for the mapping) - the arrangement NCCL's
            # own P2P transport uses.  Opening it under the exporting device's index, which is what the stock
            # tensor rebuild does, yields a mapping that kernels running on this device cannot touch.
            # The positional layout of torch's rebuild tuple is not a public interface: verify that the slot
            # patched below really is the exporter's device index before touching it.
            from torch.multiprocessing.reductions import rebuild_cuda_tensor
            fn, args = reduced
            args = list(args)
            if fn is not rebuild_cuda_tensor or len(args) < 7 or args[6] != exporter_index:
                raise RuntimeError("eet_b200.tp: torch's CUDA IPC rebuild arguments have an unexpected layout "
                                   "(storage_device is not argument 6); the fused tensor-parallel exchange cannot "
                                   "map the peers' inboxes with this torch version")
            args[6] = device.index   # storage_device
            return fn(*args)

        self.inboxes = [self.local_inbox if r == tp.rank else open_on_my_device(*h) for r, h in enumerate(everyone)]
        torch.cuda.synchronize(device)
        dist.barrier(group=tp.group)
        self._n = n
        self.inbox_ptrs = (ctypes.c_void_p * tp.size)(*[t.data_ptr() for t in self.inboxes])
        self.argmax_ptrs = (ctypes.c_void_p * tp.size)(*[t.data_ptr() + 4 * sum_words for t in self.inboxes])

    def clear_local(self):
        """Zeroes this rank's partial sums, inbox and epoch counters (see TensorParallel.reset_peer_buffers)."""
        self.local_sums.zero_()
        self.local_inbox.zero_()
        self.epochs.zero_()
        self.argmax_epochs.zero_()

    def buffer(self, which, rows):
        """This rank's partial-sum buffer 0 (attention output projection) or 1 (FFN down projection)."""
        return self.local_sums[which * self._n: which * self._n + rows * self.hidden].view(rows, self.hidden)


def init_from_env(backend="nccl"):
    """Initialises torch.distributed from the torchrun environment (RANK, WORLD_SIZE, LOCAL_RANK,
    MASTER_ADDR, MASTER_PORT), binds this process to its GPU and returns a TensorParallel over the world
    group; returns None when WORLD_SIZE is 1 or unset."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, **kwargs)
    return TensorParallel()


def head_range(num_heads, rank, size):
    """Heads [lo, hi) owned by `rank`: attention shards by whole heads, equally."""
    if num_heads % size:
        raise ValueError(f"{num_heads} heads do not divide over {size} ranks")
    per = num_heads // size
    return rank * per, (rank + 1) * per


def ff_range(d_ff, rank, size):
    """FFN inner channels [lo, hi) owned by `rank`.  The tensor-core GEMMs work in strips of 128 output
    channels (the packed layout in tiles of 64), so the split is by 128-channel strips when d_ff allows it,
    else by 64-channel tiles, and may be uneven: LLaMA-7B's 11008 = 86 strips over 8 ranks gives shards of 10
    or 11 strips."""
    if d_ff % 64:
        raise ValueError(f"d_ff {d_ff} must be a multiple of 64")
    unit = 128 if d_ff % 128 == 0 and d_ff // 128 >= size else 64
    units = d_ff // unit
    if units < size:
        raise ValueError(f"d_ff {d_ff} has fewer 64-channel tiles than the {size} ranks")
    return unit * (units * rank // size), unit * (units * (rank + 1) // size)


def vocab_range(vocab, rank, size):
    """Vocabulary columns [lo, hi) of the lm_head owned by `rank`: whole 128-column strips (the unit of the
    tensor-core GEMMs that compute prompt logits) when the vocabulary allows it, else 64-column tiles of the packed
    weight; unevenly when they do not divide (32000 = 250 strips over 8 ranks gives 31 or 32 strips per rank)."""
    if vocab % 64:
        raise ValueError(f"vocabulary size {vocab} must be a multiple of 64 for an int8 lm_head")
    unit = 128 if vocab % 128 == 0 and vocab // 128 >= size else 64
    units = vocab // unit
    if units < size:
        raise ValueError(f"vocabulary of {vocab} has fewer 64-column tiles than the {size} ranks")
    return unit * (units * rank // size), unit * (units * (rank + 1) // size)


def shard_plan(num_heads, d_ff, size):
    """Per-rank (head range, ffn range) for a tensor-parallel degree; raises if it cannot be sharded."""
    return [(head_range(num_heads, r, size), ff_range(d_ff, r, size)) for r in range(size)]
