"""CPU oracle for the Gated DeltaNet-2 forward and serving path.

TEST INFRASTRUCTURE, NOT PRODUCT. Only the test-suite, the smoke check and the
benchmark's CPU-baseline legs may import this module; the shipped package never
does and has no CPU path of its own.

This is a restatement, in plain PyTorch on the host, of the arithmetic the
reference project defines for the path. Each function names the reference
source it follows (paths are relative to the reference project's root):

* :func:`recurrence`            gdn2/reference.py:56-107   (``recurrent_gdn2``)
* :func:`chunk_cumsum`          gdn2/reference.py:110-113  (``_chunk_local_cumsum``)
* :func:`strict_tril_pairwise`  gdn2/reference.py:116-165  (``_strict_tril_kkt``)
* :func:`chunkwise`             gdn2/reference.py:168-261  (``chunk_gdn2_torch``)
* :func:`chunk_factors`         gdn2/reference.py:304-347  (forward part of
  ``forward_intermediates``) and tests/test_pipeline_simulation.py:28-100
* :func:`decode`                gdn2/inference.py:337-345  (host branch of ``gdn2_decode``)
* :func:`prefill`               gdn2/inference.py:521-539  (host branch of ``gdn2_prefill``)
* :func:`attention`             gdn2/attention.py:147-164  (pad, dispatch, slice)

Parity of this restatement with the reference is pinned by the fixtures under
``tests/golden`` (outputs of the reference's own functions, produced by
``tests/golden/make_golden.py``) and by the reference's self-consistency
properties re-stated in ``tests/test_oracle.py``.

Everything runs in one working precision (``torch.float32`` by default, as the
reference does; ``torch.float64`` is offered for tighter cross-checks).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

__all__ = [
    "make_inputs",
    "recurrence",
    "chunk_cumsum",
    "strict_tril_pairwise",
    "chunk_factors",
    "chunkwise",
    "decode",
    "prefill",
    "attention",
    "max_abs_err",
    "rel_fro_err",
    "rel_max_err",
]


# --------------------------------------------------------------------------- inputs / metrics


def make_inputs(B, S, H, DK, DV, seed=0, gate="logsigmoid16", decay_scale=4.0, dtype=torch.float32):
    """Seeded synthetic inputs, drawn on the host in the order q, k, v, g, b, w.

    ``gate="logsigmoid16"`` gives the benchmark distribution
    ``g = logsigmoid(N(0,1)) / 16``; ``gate="softplus"`` gives the one the
    reference's tests draw, ``g = -softplus(N(0,1)) * decay_scale``
    (tests/test_gdn2.py:24-35). q and k are L2-normalised per head per token,
    b and w are sigmoids of normals.
    """
    gen = torch.Generator(device="cpu").manual_seed(seed)
    kw = dict(generator=gen, dtype=torch.float32)
    q = F.normalize(torch.randn(B, S, H, DK, **kw), dim=-1)
    k = F.normalize(torch.randn(B, S, H, DK, **kw), dim=-1)
    v = torch.randn(B, S, H, DV, **kw)
    r = torch.randn(B, S, H, DK, **kw)
    if gate == "logsigmoid16":
        g = F.logsigmoid(r) / 16.0
    elif gate == "softplus":
        g = -F.softplus(r) * decay_scale
    else:
        raise ValueError(f"unknown gate distribution {gate!r}")
    b = torch.sigmoid(torch.randn(B, S, H, DK, **kw))
    w = torch.sigmoid(torch.randn(B, S, H, DV, **kw))
    q, k, v, b, w = (t.to(dtype) for t in (q, k, v, b, w))
    return q, k, v, g, b, w


def max_abs_err(a, ref):
    return (a.double() - ref.double()).abs().max().item()


def rel_fro_err(a, ref):
    """``||a - ref||_F / ||ref||_F``."""
    ref = ref.double()
    return ((a.double() - ref).norm() / ref.norm().clamp_min(1e-30)).item()


def rel_max_err(a, ref):
    """The reference tests' metric: ``max|a-ref| / max|ref|`` (tests/test_gdn2.py:38-39)."""
    ref = ref.double()
    return ((a.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()


# --------------------------------------------------------------------------- definition


def recurrence(q, k, v, g, b, w, scale=None, initial_state=None, dtype=torch.float32):
    """Token-by-token definition. Returns ``(o [B,T,H,DV], final_state [B,H,DK,DV])``.

    Per step: decay the state rows by ``exp(g_t)``, read it with the erase row
    ``b_t*k_t``, form ``u = w_t*v_t - read``, add the rank-1 write ``k_t u^T``,
    then read the output with ``scale*q_t``.
    """
    B, T, H, DK = q.shape
    DV = v.shape[-1]
    scale = DK**-0.5 if scale is None else scale
    q, k, v, g, b, w = (x.to(dtype) for x in (q, k, v, g, b, w))
    S = torch.zeros(B, H, DK, DV, dtype=dtype) if initial_state is None else initial_state.to(dtype).clone()
    o = torch.empty(B, T, H, DV, dtype=dtype)
    for t in range(T):
        S = S * g[:, t].exp().unsqueeze(-1)
        u = w[:, t] * v[:, t] - torch.einsum("bhkd,bhk->bhd", S, b[:, t] * k[:, t])
        S = S + k[:, t].unsqueeze(-1) * u.unsqueeze(-2)
        o[:, t] = torch.einsum("bhkd,bhk->bhd", S, q[:, t] * scale)
    return o, S


# --------------------------------------------------------------------------- chunkwise WY form


def chunk_cumsum(g, chunk_size):
    """Inclusive prefix sum of ``g`` restarted at every chunk boundary. ``[B,T,H,D]``."""
    B, T, H, D = g.shape
    return g.reshape(B, T // chunk_size, chunk_size, H, D).cumsum(dim=2).reshape(B, T, H, D)


def strict_tril_pairwise(left, right, G, sub_chunk_size):
    """``M[r,s] = sum_c left[r,c] * right[s,c] * exp(G[r,c]-G[s,c])`` for ``r > s``, else 0.

    Evaluated block-wise so that no exponent is ever positive: blocks left of
    the diagonal are factorised through the decay at the first row of their
    row-sub-block; diagonal sub-blocks use the exact pairwise difference.
    ``left, right, G``: ``[..., BS, D]``; returns ``[..., BS, BS]``.
    """
    *lead, BS, D = left.shape
    BC = sub_chunk_size
    n = BS // BC
    L = left.reshape(*lead, n, BC, D)
    R = right.reshape(*lead, n, BC, D)
    Gs = G.reshape(*lead, n, BC, D)
    out = left.new_zeros(*lead, n, BC, n, BC)
    strictly_lower = torch.ones(BC, BC, dtype=torch.bool).tril(-1)
    for i in range(n):
        ref = Gs[..., i, 0:1, :]
        row = L[..., i, :, :] * (Gs[..., i, :, :] - ref).exp()
        for j in range(i):
            col = R[..., j, :, :] * (ref - Gs[..., j, :, :]).exp()
            out[..., i, :, j, :] = row @ col.transpose(-1, -2)
        diff = (Gs[..., i, :, None, :] - Gs[..., i, None, :, :]).clamp_max(0)
        blk = torch.einsum("...rd,...sd,...rsd->...rs", L[..., i, :, :], R[..., i, :, :], diff.exp())
        out[..., i, :, i, :] = blk.masked_fill(~strictly_lower, 0.0)
    return out.reshape(*lead, BS, BS)


def chunk_factors(q, k, v, g, b, w, scale=None, chunk_size=64, sub_chunk_size=16, dtype=torch.float32):
    """Every chunk-local quantity of the WY form, laid out ``[B, H, NC, BS, .]``.

    Returns a dict with ``G`` (natural-log cumulative decay), ``Aqk`` (lower
    triangular incl. diagonal, scale folded in), ``Tm`` (strictly lower),
    ``Ai = (I+Tm)^-1``, ``W = Ai E``, ``U = Ai (w*v)``, ``KG`` (``k`` carried to
    the chunk end), ``Qg`` (``scale*q*gamma``) and ``gamma_last`` ``[B,H,NC,DK]``.
    """
    B, T, H, DK = q.shape
    BS = chunk_size
    if T % BS:
        raise ValueError(f"sequence length {T} must be divisible by chunk_size {BS}")
    if BS % sub_chunk_size:
        raise ValueError(f"chunk_size {BS} must be divisible by sub_chunk_size {sub_chunk_size}")
    scale = DK**-0.5 if scale is None else scale
    NC = T // BS
    q, k, v, g, b, w = (x.to(dtype) for x in (q, k, v, g, b, w))

    def blk(x):
        return x.reshape(B, NC, BS, H, x.shape[-1]).permute(0, 3, 1, 2, 4)

    G = blk(chunk_cumsum(g, BS))
    qb, kb, vb, bb, wb = blk(q), blk(k), blk(v), blk(b), blk(w)
    gamma = G.exp()
    E = bb * kb * gamma
    Z = wb * vb
    Tm = strict_tril_pairwise(bb * kb, kb, G, sub_chunk_size)
    eye = torch.eye(BS, dtype=dtype).expand_as(Tm)
    Ai = torch.linalg.solve_triangular(eye + Tm, eye, upper=False, unitriangular=True)
    Aqk = strict_tril_pairwise(qb, kb, G, sub_chunk_size)
    Aqk = (Aqk + torch.diag_embed((qb * kb).sum(-1))) * scale
    return dict(
        G=G, Aqk=Aqk, Tm=Tm, Ai=Ai, W=Ai @ E, U=Ai @ Z,
        KG=kb * (G[..., -1:, :] - G).exp(), Qg=qb * gamma * scale, gamma_last=gamma[..., -1, :],
    )


def chunkwise(q, k, v, g, b, w, scale=None, initial_state=None, chunk_size=64, sub_chunk_size=16,
              dtype=torch.float32, return_chunk_states=False):
    """Chunkwise WY evaluation. Returns ``(o, final_state)`` or ``(o, final_state, h)``.

    ``h [B, NC, H, DK, DV]`` holds the state entering every chunk (what the
    reference's scan kernel snapshots, gdn2/forward.py:617-620).
    """
    B, T, H, DK = q.shape
    DV = v.shape[-1]
    f = chunk_factors(q, k, v, g, b, w, scale, chunk_size, sub_chunk_size, dtype)
    NC = T // chunk_size
    S = torch.zeros(B, H, DK, DV, dtype=dtype) if initial_state is None else initial_state.to(dtype).clone()
    o = torch.empty(B, H, NC, chunk_size, DV, dtype=dtype)
    h = torch.empty(B, NC, H, DK, DV, dtype=dtype) if return_chunk_states else None
    for n in range(NC):
        if h is not None:
            h[:, n] = S
        Un = f["U"][:, :, n] - f["W"][:, :, n] @ S
        o[:, :, n] = f["Qg"][:, :, n] @ S + f["Aqk"][:, :, n] @ Un
        S = f["gamma_last"][:, :, n].unsqueeze(-1) * S + f["KG"][:, :, n].transpose(-1, -2) @ Un
    o = o.permute(0, 2, 3, 1, 4).reshape(B, T, H, DV)
    return (o, S, h) if return_chunk_states else (o, S)


# --------------------------------------------------------------------------- serving


def decode(q, k, v, g, b, w, state, scale=None):
    """``n`` recurrence steps on ``[B,n,H,D]`` tokens; ``state`` is updated in place.

    Returns ``o [B,n,H,DV]`` in ``v.dtype``; arithmetic in the state's dtype.
    """
    B, n, H, DK = q.shape
    scale = DK**-0.5 if scale is None else scale
    dt = state.dtype
    outs = []
    for t in range(n):
        state.mul_(g[:, t].to(dt).exp().unsqueeze(-1))
        u = (w[:, t] * v[:, t]).to(dt) - torch.einsum("bhkd,bhk->bhd", state, (b[:, t] * k[:, t]).to(dt))
        state.add_(k[:, t].to(dt).unsqueeze(-1) * u.unsqueeze(-2))
        outs.append(torch.einsum("bhkd,bhk->bhd", state, q[:, t].to(dt) * scale))
    return torch.stack(outs, dim=1).to(v.dtype)


def prefill(q, k, v, g, b, w, state=None, scale=None, chunk_size=64, sub_chunk_size=16):
    """Whole chunks through :func:`chunkwise`, the ragged tail through :func:`decode`."""
    B, S, H, DK = q.shape
    DV = v.shape[-1]
    scale = DK**-0.5 if scale is None else scale
    n_full = (S // chunk_size) * chunk_size
    state = torch.zeros(B, H, DK, DV) if state is None else state.to(torch.float32).contiguous()
    outs = []
    if n_full:
        o1, state = chunkwise(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, state, chunk_size, sub_chunk_size)
        outs.append(o1)
    if S > n_full:
        outs.append(decode(*(t[:, n_full:] for t in (q, k, v, g, b, w)), state, scale).to(torch.float32))
    return torch.cat(outs, dim=1), state


def attention(q, k, v, g, b, w, scale=None, initial_state=None, chunk_size=64, sub_chunk_size=16):
    """Pad the sequence with inert tokens (``g=0, b=w=0``) to a chunk multiple, run
    :func:`chunkwise`, slice back. Returns ``(o, final_state)``."""
    S = q.shape[1]
    S_pad = math.ceil(S / chunk_size) * chunk_size
    if S_pad != S:
        q, k, v, g, b, w = (F.pad(x, (0, 0, 0, 0, 0, S_pad - S)) for x in (q, k, v, g, b, w))
    o, s = chunkwise(q, k, v, g, b, w, scale, initial_state, chunk_size, sub_chunk_size)
    return o[:, :S], s
