"""Head-parallel GatedDeltaNet2 over the ranks of one ``torch.distributed`` process group.

Every (batch, head) pair of the recurrence is independent, so the attention kernels need no
communication: rank ``r`` of ``W`` owns key heads ``[r*HK/W, (r+1)*HK/W)`` and the value heads that
read them. The projections feeding the kernels are column-sharded (rows of the ``nn.Linear``
weights), the short convolutions, ``A_log`` and ``dt_bias`` are sliced by channel / head,
``o_norm.weight`` is replicated, ``o_proj`` is row-sharded (columns of its weight), and the partial
outputs are summed with ONE all-reduce per call (NCCL over NVLink on GPUs, gloo in CPU tests).
The cache is sharded the same way: each rank keeps ``recurrent_state [B, H/W, DK, DV]`` and its
own conv channels.

The reference project has no multi-device code; this is the sharding its layer admits
(gdn2/attention.py:232-297: per-head projections, ``head_repeat`` expansion).
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch
import torch.distributed as dist

from .attention import GatedDeltaNet2
from .config import GatedDeltaNet2Config

__all__ = ["shard_config", "shard_state_dict", "TensorParallelGatedDeltaNet2", "FusedOutputReduce"]


def shard_config(cfg: GatedDeltaNet2Config, world: int) -> GatedDeltaNet2Config:
    """Per-rank config: head counts divided by ``world``, everything else unchanged."""
    H = cfg.num_heads
    HK = cfg.num_kv_heads or H
    if HK % world or H % world:
        raise ValueError(f"num_kv_heads {HK} and num_heads {H} must be divisible by the world size {world}")
    return dataclasses.replace(cfg, num_heads=H // world, num_kv_heads=HK // world)


def shard_state_dict(sd: dict, cfg: GatedDeltaNet2Config, rank: int, world: int) -> dict:
    """Slice a full-layer ``state_dict`` down to what rank ``rank`` of ``world`` owns."""
    H = cfg.num_heads
    HK = cfg.num_kv_heads or H
    DK = cfg.head_dim_k
    DV = cfg.head_dim_v or DK
    shard_config(cfg, world)
    qk = slice(rank * (HK // world) * DK, (rank + 1) * (HK // world) * DK)
    vv = slice(rank * (H // world) * DV, (rank + 1) * (H // world) * DV)
    hk = slice(rank * (HK // world), (rank + 1) * (HK // world))
    out = {}
    for name, t in sd.items():
        base = name.split(".")[0]
        if base in ("q_proj", "k_proj", "b_proj", "f_proj", "q_conv", "k_conv"):
            out[name] = t[qk].clone()
        elif base in ("v_proj", "w_proj", "o_gate_proj", "v_conv"):
            out[name] = t[vv].clone()
        elif base == "o_proj":
            out[name] = t[:, vv].clone()
        elif base in ("A_log", "dt_bias"):
            out[name] = t[hk].clone()
        else:   # o_norm.weight: per value channel inside a head, identical on every rank
            out[name] = t.clone()
    return out


class FusedOutputReduce:
    """``o_proj`` + sum over ranks in ONE kernel per rank (``gdn2_oproj_reduce``) for decode-sized inputs.

    Every rank allocates the exchange buffer from PyTorch's symmetric-memory allocator, which maps it into all
    peers' address spaces; the kernel writes its fp32 partial sums into every peer's buffer with ordinary stores
    over NVLink and adds the partials that arrive in its own. Construction is collective (every rank of the group
    must do it, in the same order); afterwards a call is one kernel launch with no host-side rendezvous, so it
    can be captured in a CUDA graph.
    """

    MAX_ROWS = 8

    def __init__(self, hidden: int, device, group=None, wait_cycles: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi

        self.K = _cabi.kernels()
        self.group = dist.group.WORLD if group is None else group
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.hidden, self.wait_cycles = hidden, wait_cycles
        off = ctypes.c_size_t(0)
        nbytes = self.K.lib.gdn2_oproj_reduce_buffer_bytes(self.world, hidden, ctypes.byref(off))
        if nbytes == 0:
            raise ValueError(f"hidden size {hidden} must be a multiple of 32")
        self.buf = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_slots = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.peer_flags = torch.tensor([p + off.value for p in ptrs], dtype=torch.int64, device=device)
        self.epochs = torch.zeros(hidden // 32, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                   # every rank's buffer is zeroed before anyone writes into it

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x [rows <= 8, K]`` (this rank's slice), ``weight [hidden, K]`` -> ``[rows, hidden]`` summed over ranks."""
        if out is None:
            out = torch.empty(x.shape[0], self.hidden, dtype=x.dtype, device=x.device)
        return self.K.oproj_reduce(x, weight, out, self.peer_slots, self.peer_flags, self.epochs, self.rank,
                                   self.world, self.wait_cycles)


class TensorParallelGatedDeltaNet2(GatedDeltaNet2):
    """One rank's shard of the layer; ``forward`` / ``prefill`` / ``decode`` / ``step`` return the
    full ``[B, S, hidden]`` output on every rank after the sum over ranks: one all-reduce after ``o_proj``, or,
    once ``enable_fused_reduce()`` has been called, ``o_proj`` and the sum in one kernel for calls of at most 8
    token rows (the one-token step)."""

    def __init__(self, full_config: GatedDeltaNet2Config, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.full_cfg = full_config
        self.fused_reduce = None
        super().__init__(shard_config(full_config, self.world))

    def load_full_state_dict(self, sd: dict):
        """Load this rank's slice of a full (unsharded) ``state_dict``."""
        return self.load_state_dict(shard_state_dict(sd, self.full_cfg, self.rank, self.world))

    def enable_fused_reduce(self, wait_cycles: int = 0):
        """Collective over the group: set up the exchange buffers of the fused ``o_proj`` + sum kernel. Call it
        on every rank once the layer sits on its CUDA device."""
        if self.world > 1:
            self.fused_reduce = FusedOutputReduce(self.cfg.hidden_size, self.o_proj.weight.device, self.group, wait_cycles)
        return self

    def _project_out(self, normed):
        B, S, K = normed.shape
        w = self.o_proj.weight
        if (self.fused_reduce is not None and B * S <= FusedOutputReduce.MAX_ROWS and self.o_proj.bias is None
                and normed.dtype == w.dtype and B * S * K * w.element_size() <= 64 * 1024):
            return self.fused_reduce(normed.reshape(B * S, K), w).view(B, S, -1)
        y = self.o_proj(normed)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
