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

import dataclasses

import torch
import torch.distributed as dist

from .attention import GatedDeltaNet2
from .config import GatedDeltaNet2Config

__all__ = ["shard_config", "shard_state_dict", "TensorParallelGatedDeltaNet2"]


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


class TensorParallelGatedDeltaNet2(GatedDeltaNet2):
    """One rank's shard of the layer; ``forward`` / ``prefill`` / ``decode`` / ``step`` return the
    full ``[B, S, hidden]`` output on every rank after the all-reduce."""

    def __init__(self, full_config: GatedDeltaNet2Config, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.full_cfg = full_config
        super().__init__(shard_config(full_config, self.world))

    def load_full_state_dict(self, sd: dict):
        """Load this rank's slice of a full (unsharded) ``state_dict``."""
        return self.load_state_dict(shard_state_dict(sd, self.full_cfg, self.rank, self.world))

    def _reduce(self, y):
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
