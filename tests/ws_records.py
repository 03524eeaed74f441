"""Decode the chunk-local stage's workspace records (tensor-core family, DK = DV = 128, bf16) back into
the matrices they hold, laid out like the oracle's ``chunk_factors``: ``[B, H, NC, 64, .]``.

Test helper. The record formats are the ones ``include/gdn2_b200.h`` documents beside
``gdn2_prefill_workspace_layout``.
"""

from __future__ import annotations

import torch

BS, D, VAL_SCALE = 64, 128, 256.0


def decode_tc_workspace(ws: torch.Tensor, layout: dict, B: int, S: int, H: int, HK: int | None = None) -> dict:
    """``ws``: the uint8 workspace tensor (any device); ``layout``: ``NativeKernels.workspace_layout``.
    ``H`` value heads (records ``U``), ``HK`` key heads (every other record; default ``H``)."""
    NC = S // BS
    HK = HK or H
    nch = B * HK * NC
    raw = ws.cpu()

    def records(off, nbytes, dtype, count=nch):
        return raw[off: off + count * nbytes].view(dtype).reshape(count, -1)

    # WQ: bf16 [dk/8][128 rows][8] -> [rows, dk]
    wq = records(layout["wq"], 2 * BS * D * 2, torch.bfloat16).reshape(nch, D // 8, 2 * BS, 8)
    wq = wq.permute(0, 2, 1, 3).reshape(nch, 2 * BS, D).float()
    # AQK: fp16 [s/8][64 r][8] -> [r, s], stored times 256
    aqk = records(layout["aqk"], BS * BS * 2, torch.float16).reshape(nch, BS // 8, BS, 8)
    aqk = aqk.permute(0, 2, 1, 3).reshape(nch, BS, BS).float() / VAL_SCALE
    # KG^T: fp16 [t/8][128 dk][8] -> [t, dk], stored times 256
    kgt = records(layout["kgt"], D * BS * 2, torch.float16).reshape(nch, BS // 8, D, 8)
    kg = kgt.permute(0, 1, 3, 2).reshape(nch, BS, D).float() / VAL_SCALE
    # U^T: fp16 [t/8][128 dv][8] -> [t, dv], stored divided by 256
    nch_v = B * H * NC
    ut = records(layout["ut"], D * BS * 2, torch.float16, nch_v).reshape(nch_v, BS // 8, D, 8)
    u = ut.permute(0, 1, 3, 2).reshape(nch_v, BS, D).float() * VAL_SCALE
    gl = records(layout["gl"], D * 4, torch.float32)
    flags = raw[layout["flags"]: layout["flags"] + nch * 4].view(torch.int32)

    def shaped(x, heads=HK):
        return x.reshape(B, heads, NC, *x.shape[1:])

    return dict(W=shaped(wq[:, :BS]), Qg=shaped(wq[:, BS:]), Aqk=shaped(aqk), KG=shaped(kg), U=shaped(u, H),
                gamma_last=shaped(gl), flags=shaped(flags))
