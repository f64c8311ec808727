"""Autograd wrappers of the memory-bound sm_100a kernels: RMSNorm / LayerNorm (residual add fused),
RoPE on the packed QKV projection, SwiGLU / GeGLU / GELU, vocab-parallel embedding and cross-entropy.

Each op takes the CUDA kernel when its input lives on a GPU and the plain-PyTorch restatement of the
same math (the numerical oracle of the tests, and the CPU/gloo plumbing path) otherwise.
"""
from __future__ import annotations

import math
from functools import lru_cache

import torch
import torch.distributed as dist

from . import _lib

_NORM_PARTS = 296  # CTAs (and partial rows) of the norm backward


# --------------------------------------------------------------------------------------------
# Norms
# --------------------------------------------------------------------------------------------
def _norm_ref(h, w, b, eps, rms):
    hf = h.float()
    if rms:
        y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    else:
        y = torch.nn.functional.layer_norm(hf, (h.shape[-1],), w.float(), None if b is None else b.float(), eps)
    return y.to(h.dtype)


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, b, eps, rms):
        lib = _lib.load()
        rows, H = x.shape
        y = torch.empty_like(x)
        h = torch.empty_like(x) if residual is not None else x
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = lib.hg_norm_fwd(x.data_ptr(), _lib.ptr(residual), w.data_ptr(), _lib.ptr(b), y.data_ptr(),
                             h.data_ptr() if residual is not None else 0, rstd.data_ptr(), _lib.ptr(mean), rows, H,
                             float(eps), int(rms), _lib.stream())
        _lib.check(rc, "hg_norm_fwd")
        _lib.count_launch()
        ctx.save_for_backward(h, w, rstd, mean if mean is not None else rstd)
        ctx.rms, ctx.has_res, ctx.has_bias = rms, residual is not None, b is not None
        if residual is None:
            return y
        return y, h

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, w, rstd, mean = ctx.saved_tensors
        lib = _lib.load()
        rows, H = h.shape
        dy = dy.contiguous()
        dres = dh.contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        parts = _NORM_PARTS
        partial = torch.empty((2 if not ctx.rms else 1) * parts * H, dtype=torch.float32, device=h.device)
        mgw = getattr(w, "main_grad", None)
        dw = mgw if mgw is not None else torch.empty(H, dtype=torch.float32, device=h.device)
        db = None
        if ctx.has_bias:
            # zero-filled: the kernel's accumulate switch is shared with dw (which may add into main_grad)
            db = torch.zeros(H, dtype=torch.float32, device=h.device)
        rc = lib.hg_norm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                             0 if ctx.rms else mean.data_ptr(), _lib.ptr(dres), dx.data_ptr(), dw.data_ptr(),
                             _lib.ptr(db), partial.data_ptr(), parts, rows, H, int(ctx.rms),
                             1 if (mgw is not None and not getattr(w, "mg_fresh", False)) else 0, _lib.stream())
        if mgw is not None:
            w.mg_fresh = False
        _lib.check(rc, "hg_norm_bwd")
        _lib.count_launch(2 if ctx.rms else 3)
        gw = None if mgw is not None else dw.to(w.dtype)
        gb = db.to(w.dtype) if db is not None else None
        # dx carries the gradient of both x and the residual input (they are summed in the forward)
        return dx, (dx if ctx.has_res else None), gw, gb, None, None


def norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, eps: float = 1e-5, rms: bool = True,
         residual: torch.Tensor | None = None):
    """Returns ``(normalised, h)`` with ``h = x + residual`` (``h is x`` without a residual).

    Fusing the residual add means the block computes ``h = x + attn_out`` and ``norm(h)`` in one pass
    over memory.  Note for LayerNorm with bias: the bias gradient is returned through the normal
    autograd path (fp32 -> parameter dtype)."""
    shp = x.shape
    if not x.is_cuda:
        h = x if residual is None else x + residual
        return _norm_ref(h, w, b, eps, rms), h
    x2 = x.reshape(-1, shp[-1]).contiguous()
    r2 = residual.reshape(-1, shp[-1]).contiguous() if residual is not None else None
    if r2 is None:
        return _Norm.apply(x2, None, w, b, eps, rms).view(shp), x
    y, h = _Norm.apply(x2, r2, w, b, eps, rms)
    return y.view(shp), h.view(shp)


# --------------------------------------------------------------------------------------------
# RoPE
# --------------------------------------------------------------------------------------------
_ROPE_CACHE: dict = {}


def llama3_scale_inv_freq(inv: torch.Tensor, factor: float = 8.0, low_freq_factor: float = 1.0,
                          high_freq_factor: float = 4.0, original_max_pos: int = 8192) -> torch.Tensor:
    """Llama-3.x frequency scaling: wavelengths beyond ``original_max_pos / low_freq_factor`` are stretched by
    ``factor``, those below ``original_max_pos / high_freq_factor`` are kept, the band in between is blended
    (galvatron/core/runtime/transformer/rotary_pos_embedding.py:124-157)."""
    import math

    wavelen = 2 * math.pi / inv
    low_wl, high_wl = original_max_pos / low_freq_factor, original_max_pos / high_freq_factor
    out = torch.where(wavelen > low_wl, inv / factor, inv)
    smooth = (original_max_pos / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1 - smooth) * inv / factor + smooth * inv
    medium = ~(wavelen < high_wl) & ~(wavelen > low_wl)
    return torch.where(medium, blended, out)


def rope_tables(max_pos: int, rot_dim: int, base: float, device: str, interp: float = 1.0, llama3_factor: float = 0.0):
    """fp32 ``cos``/``sin`` tables ``[max_pos, rot_dim/2]`` (inv_freq = base^(-2i/dim), positions / interp; optional
    Llama-3 frequency scaling).  Cached per argument tuple: every layer of a model shares one pair."""
    key = (max_pos, rot_dim, float(base), str(device), float(interp), float(llama3_factor or 0.0))
    hit = _ROPE_CACHE.get(key)
    if hit is not None:
        return hit
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    if llama3_factor:
        inv = llama3_scale_inv_freq(inv, llama3_factor)
    pos = torch.arange(max_pos, dtype=torch.float32) / interp
    f = torch.outer(pos, inv)
    out = (f.cos().to(device).contiguous(), f.sin().to(device).contiguous())
    if len(_ROPE_CACHE) > 64:
        _ROPE_CACHE.clear()
    _ROPE_CACHE[key] = out
    return out


def _rope_ref(t, cos, sin, pos, sign=1.0, interleaved=False):
    # t: [tokens, heads, hd]; rotate-half (or interleaved pairs) on the first 2*half channels
    half = cos.shape[1]
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :] * sign
    out = t.clone()
    if interleaved:
        a, b = t[..., 0:2 * half:2].float(), t[..., 1:2 * half:2].float()
        out[..., 0:2 * half:2] = (a * c - b * s).to(t.dtype)
        out[..., 1:2 * half:2] = (b * c + a * s).to(t.dtype)
        return out
    a, b = t[..., :half].float(), t[..., half:2 * half].float()
    out[..., :half] = (a * c - b * s).to(t.dtype)
    out[..., half:2 * half] = (b * c + a * s).to(t.dtype)
    return out


class _RopeInplace(torch.autograd.Function):
    """Rotates the listed head slots of a ``[tokens, slots*hd]`` buffer in place."""

    @staticmethod
    def forward(ctx, buf, head_off, cos, sin, batch, pos, pos_offset, rot_dim, interleaved=False):
        ctx.args = (head_off, cos, sin, batch, pos, pos_offset, rot_dim, interleaved)
        _rope_launch(buf, head_off, cos, sin, batch, pos, pos_offset, rot_dim, False, interleaved)
        ctx.mark_dirty(buf)
        return buf

    @staticmethod
    def backward(ctx, g):
        head_off, cos, sin, batch, pos, pos_offset, rot_dim, interleaved = ctx.args
        # the incoming gradient buffer is produced by the attention backward for this op alone, so it is
        # rotated back in place
        if not g.is_contiguous():
            g = g.contiguous()
        _rope_launch(g, head_off, cos, sin, batch, pos, pos_offset, rot_dim, True, interleaved)
        return g, None, None, None, None, None, None, None, None


def _rope_launch(buf, head_off, cos, sin, batch, pos, pos_offset, rot_dim, backward, interleaved=False):
    lib = _lib.load()
    tokens, pitch = buf.shape
    rc = lib.hg_rope(buf.data_ptr(), head_off.data_ptr(), head_off.numel(), pitch, tokens, batch, _lib.ptr(pos),
                     pos_offset, cos.data_ptr(), sin.data_ptr(), rot_dim, int(backward) | (2 if interleaved else 0), _lib.stream())
    _lib.check(rc, "hg_rope")
    _lib.count_launch()


def rope_packed(qkv: torch.Tensor, head_slots: torch.Tensor, hd: int, cos: torch.Tensor, sin: torch.Tensor,
                batch: int, pos: torch.Tensor | None = None, pos_offset: int = 0,
                interleaved: bool = False) -> torch.Tensor:
    """Apply RoPE to the head slots ``head_slots`` (int32 slot indices) of ``qkv`` ``[tokens, slots*hd]`` (token
    t = s*batch + b has position ``pos[t]`` or ``s + pos_offset``): rotate-half, or with ``interleaved`` the
    channel pairs ``(2i, 2i+1)`` (the reference's ``rotary_interleaved``, rope_utils.py:67-83)."""
    rot_dim = 2 * cos.shape[1]
    if not qkv.is_cuda:
        tokens = qkv.shape[0]
        t3 = qkv.view(tokens, -1, hd)
        if pos is None:
            p = torch.arange(tokens, device=qkv.device) // batch + pos_offset
        else:
            p = pos.long()
        out = t3.clone()
        idx = head_slots.long()
        out[:, idx] = _rope_ref(t3[:, idx], cos, sin, p, interleaved=interleaved)
        return out.view_as(qkv)
    head_off = (head_slots.to(torch.int32) * hd).contiguous()
    if pos is not None:
        pos = pos.to(torch.int32).contiguous()
    return _RopeInplace.apply(qkv, head_off, cos, sin, batch, pos, pos_offset, rot_dim, interleaved)


def mrope_angles(position_ids: torch.Tensor, mrope_section, rot_dim: int, base: float = 10000.0,
                 interp: float = 1.0) -> torch.Tensor:
    """Multimodal RoPE angles.  ``position_ids [3, B, S]`` carries a temporal, a height and a width position per
    token; the ``rot_dim / 2`` frequency channels are cut into ``mrope_section`` (e.g. ``[16, 24, 24]``) and section
    ``i`` takes its angle from position row ``i % 3``.  Returns fp32 angles ``[S, B, rot_dim / 2]`` (the two halves of
    the rotate-half layout share them).  Same channel assignment as the reference's ``MultimodalRotaryEmbedding``
    (galvatron/core/runtime/transformer/rotary_pos_embedding.py:267-353) and as Qwen2-VL."""
    if position_ids.dim() != 3 or position_ids.shape[0] != 3:
        raise ValueError("position_ids must be [3, batch, seq]")
    half = rot_dim // 2
    if sum(mrope_section) != half:
        raise ValueError("mrope_section %s must sum to rot_dim / 2 = %d" % (list(mrope_section), half))
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=position_ids.device) / rot_dim))
    ang = position_ids.to(torch.float32)[..., None] / interp * inv          # [3, B, S, half]
    parts, lo = [], 0
    for i, n in enumerate(mrope_section):
        parts.append(ang[i % 3, :, :, lo:lo + n])
        lo += n
    return torch.cat(parts, dim=-1).transpose(0, 1).contiguous()           # [S, B, half]


def apply_mrope(t: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE of ``t [S, B, heads, hd]`` by per-token ``angles [S, B, rot_dim / 2]`` (from
    :func:`mrope_angles`); channels past ``rot_dim`` pass through.  Differentiable (plain tensor ops: the vision
    position rows change per sample, so there is no table to cache)."""
    half = angles.shape[-1]
    c = angles.cos()[:, :, None, :]
    s = angles.sin()[:, :, None, :]
    a, b = t[..., :half].float(), t[..., half:2 * half].float()
    rot = torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(t.dtype)
    return torch.cat([rot, t[..., 2 * half:]], dim=-1) if t.shape[-1] > 2 * half else rot


# --------------------------------------------------------------------------------------------
# Gated activations
# --------------------------------------------------------------------------------------------
_KIND = {"swiglu": 0, "geglu": 1, "gelu": 2}


def _act_ref(y, kind):
    if kind == "gelu":
        return torch.nn.functional.gelu(y.float(), approximate="tanh").to(y.dtype)
    a, b = y.float().chunk(2, dim=-1)
    act = torch.nn.functional.silu(a) if kind == "swiglu" else torch.nn.functional.gelu(a, approximate="tanh")
    return (act * b).to(y.dtype)


class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, kind):
        lib = _lib.load()
        rows = y.shape[0]
        F = y.shape[1] if kind == 2 else y.shape[1] // 2
        out = torch.empty((rows, F), dtype=y.dtype, device=y.device)
        _lib.check(lib.hg_glu_fwd(y.data_ptr(), out.data_ptr(), rows, F, kind, _lib.stream()), "hg_glu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(y)
        ctx.kind = kind
        return out

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        lib = _lib.load()
        g = g.contiguous()
        dy = torch.empty_like(y)
        F = g.shape[1]
        _lib.check(lib.hg_glu_bwd(g.data_ptr(), y.data_ptr(), dy.data_ptr(), y.shape[0], F, ctx.kind, _lib.stream()),
                   "hg_glu_bwd")
        _lib.count_launch()
        return dy, None


def activation(y: torch.Tensor, kind: str = "swiglu") -> torch.Tensor:
    """``swiglu`` / ``geglu``: ``act(y[..., :F]) * y[..., F:]``;  ``gelu``: tanh-approximated GELU."""
    if not y.is_cuda:
        return _act_ref(y, kind)
    shp = y.shape
    out = _Glu.apply(y.reshape(-1, shp[-1]).contiguous(), _KIND[kind])
    return out.view(*shp[:-1], out.shape[-1])


# --------------------------------------------------------------------------------------------
# Embedding (vocab-parallel aware)
# --------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, W, pos_emb, v0, batch, pos_offset):
        lib = _lib.load()
        tokens = ids.numel()
        H = W.shape[1]
        out = torch.empty((tokens, H), dtype=W.dtype, device=W.device)
        _lib.check(lib.hg_embedding_fwd(ids.data_ptr(), W.data_ptr(), _lib.ptr(pos_emb), out.data_ptr(), tokens, H,
                                        v0, v0 + W.shape[0], batch, pos_offset, _lib.stream()), "hg_embedding_fwd")
        _lib.count_launch()
        ctx.save_for_backward(ids)
        ctx.W, ctx.pos_emb, ctx.args = W, pos_emb, (v0, batch, pos_offset)
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        W, pos_emb = ctx.W, ctx.pos_emb
        v0, batch, pos_offset = ctx.args
        lib = _lib.load()
        g = g.contiguous()
        mg = getattr(W, "main_grad", None)
        if mg is not None and getattr(W, "mg_fresh", False):
            mg.zero_()
            W.mg_fresh = False
        dW = mg if mg is not None else torch.zeros(W.shape, dtype=torch.float32, device=W.device)
        dpos = None
        if pos_emb is not None:
            mgp = getattr(pos_emb, "main_grad", None)
            if mgp is not None and getattr(pos_emb, "mg_fresh", False):
                mgp.zero_()
                pos_emb.mg_fresh = False
            dpos = mgp if mgp is not None else torch.zeros(pos_emb.shape, dtype=torch.float32, device=W.device)
        _lib.check(lib.hg_embedding_bwd(ids.data_ptr(), g.data_ptr(), dW.data_ptr(), _lib.ptr(dpos), ids.numel(),
                                        W.shape[1], v0, v0 + W.shape[0], batch, pos_offset, _lib.stream()),
                   "hg_embedding_bwd")
        _lib.count_launch()
        gW = None if mg is not None else dW.to(W.dtype)
        gP = None
        if pos_emb is not None and getattr(pos_emb, "main_grad", None) is None:
            gP = dpos.to(pos_emb.dtype)
        return None, gW, gP, None, None, None


def embedding(ids: torch.Tensor, W: torch.Tensor, v0: int = 0, pos_emb: torch.Tensor | None = None, batch: int = 1,
              pos_offset: int = 0) -> torch.Tensor:
    """Masked lookup ``W[id - v0]`` (zero rows for ids outside this shard) for flat ``ids`` ``[tokens]``;
    optionally adds learned absolute positions ``pos_emb[s + pos_offset]`` (token t = s*batch + b)."""
    ids = ids.reshape(-1)
    if not W.is_cuda:
        local = ids - v0
        mask = (local < 0) | (local >= W.shape[0])
        out = torch.nn.functional.embedding(local.clamp(0, W.shape[0] - 1), W)
        out = out.masked_fill(mask[:, None], 0)
        if pos_emb is not None:
            p = torch.arange(ids.numel(), device=ids.device) // batch + pos_offset
            out = out + pos_emb[p]
        return out
    return _Embedding.apply(ids.contiguous().long(), W, pos_emb, v0, batch, pos_offset)


# --------------------------------------------------------------------------------------------
# Vocab-parallel cross entropy
# --------------------------------------------------------------------------------------------
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, v0, group):
        lib = _lib.load()
        rows, V = logits.shape
        dev = logits.device
        stats = torch.empty((3, rows), dtype=torch.float32, device=dev)
        _lib.check(lib.hg_xent_stats(logits.data_ptr(), logits.stride(0), targets.data_ptr(), v0, V,
                                     stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(), rows,
                                     _lib.stream()), "hg_xent_stats")
        _lib.count_launch()
        lmax, lsum, pred = stats[0], stats[1], stats[2]
        if group is not None:
            gmax = lmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack([lsum * torch.exp(lmax - gmax), pred])
            dist.all_reduce(packed, group=group)
            gsum, pred = packed[0], packed[1]
        else:
            gmax, gsum = lmax, lsum
        loss = torch.log(gsum) + gmax - pred
        ctx.save_for_backward(logits, targets, gmax, gsum)
        ctx.v0 = v0
        return loss

    @staticmethod
    def backward(ctx, g):
        logits, targets, gmax, gsum = ctx.saved_tensors
        lib = _lib.load()
        rows, V = logits.shape
        g = g.float().contiguous()
        # the logits buffer is dead after the loss: overwrite it with its own gradient
        _lib.check(lib.hg_xent_bwd(logits.data_ptr(), logits.stride(0), targets.data_ptr(), ctx.v0, V,
                                   gmax.data_ptr(), gsum.data_ptr(), g.data_ptr(), rows, _lib.stream()),
                   "hg_xent_bwd")
        _lib.count_launch()
        return logits, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, v0: int = 0, group=None) -> torch.Tensor:
    """Per-token loss ``[rows]`` (fp32) of ``logits [rows, V_local]`` against global ``targets``; with a
    vocab-parallel ``group`` the shard statistics are combined by one MAX and one SUM all-reduce.
    The backward overwrites ``logits`` in place (the tensor must not be used afterwards)."""
    targets = targets.reshape(-1)
    from ..parallel.mappings import _pg

    group, n_ranks, _ = _pg(group)  # CommGroup / ProcessGroup / None -> ProcessGroup or None (single rank)
    if not logits.is_cuda:
        lf = logits.float()
        lmax = lf.max(-1).values.detach()  # the shift cancels analytically: it must not carry a gradient
        if group is not None:
            gmax = lmax.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        else:
            gmax = lmax
        ex = torch.exp(lf - gmax[:, None])
        local = targets - v0
        inside = (local >= 0) & (local < logits.shape[1])
        pred = torch.where(inside, lf.gather(1, local.clamp(0, logits.shape[1] - 1)[:, None])[:, 0],
                           torch.zeros_like(gmax))
        ssum = ex.sum(-1)
        if group is not None:
            from ..parallel.mappings import all_reduce_sum

            packed = all_reduce_sum(torch.stack([ssum, pred]), group)
            ssum, pred = packed[0], packed[1]
        return torch.log(ssum) + gmax - pred
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    return _CrossEntropy.apply(logits, targets.contiguous().long(), v0, group)


# ---- top-k router ---------------------------------------------------------------------------------------------
ROUTER_MODES = {("softmax", False): 0, ("softmax", True): 1, ("sigmoid", False): 2, ("sigmoid", True): 2}


class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, mode, scaling):
        lib = _lib.load()
        T, E = logits.shape
        dev = logits.device
        probs = torch.empty((T, k), dtype=torch.float32, device=dev)
        idx = torch.empty((T, k), dtype=torch.int32, device=dev)
        scores = torch.empty((T, E), dtype=torch.float32, device=dev)
        counts = torch.zeros(E, dtype=torch.float32, device=dev)
        rc = lib.hg_router_topk_fwd(logits.data_ptr(), _lib.ptr(bias), T, E, k, mode, float(scaling), probs.data_ptr(),
                                    idx.data_ptr(), scores.data_ptr(), counts.data_ptr(), _lib.stream())
        _lib.check(rc, "hg_router_topk_fwd")
        _lib.count_launch()
        ctx.save_for_backward(scores, probs, idx)
        ctx.k, ctx.mode, ctx.scaling = k, mode, scaling
        ctx.mark_non_differentiable(idx, counts)
        return probs, idx, scores, counts

    @staticmethod
    def backward(ctx, dprobs, _didx, dscores, _dcounts):
        scores, probs, idx = ctx.saved_tensors
        lib = _lib.load()
        T, E = scores.shape
        dlogits = torch.empty_like(scores)
        dprobs = dprobs.contiguous().float()
        ds = dscores.contiguous().float() if dscores is not None else None
        rc = lib.hg_router_topk_bwd(scores.data_ptr(), probs.data_ptr(), idx.data_ptr(), dprobs.data_ptr(), _lib.ptr(ds), T,
                                    E, ctx.k, ctx.mode, float(ctx.scaling), dlogits.data_ptr(), _lib.stream())
        _lib.check(rc, "hg_router_topk_bwd")
        _lib.count_launch()
        return dlogits, None, None, None, None


def router_topk(logits: torch.Tensor, k: int, score: str = "softmax", pre_softmax: bool = False,
                bias: torch.Tensor | None = None, scaling: float | None = None):
    """``logits [T, E]`` fp32 -> ``(probs [T, k] fp32, idx [T, k] int64, scores [T, E] fp32, counts [E] fp32)``.

    One kernel per direction on CUDA (E <= 256, k <= 8); ``scores`` is the full softmax / sigmoid (differentiable,
    for the load-balancing losses) and ``counts`` the number of tokens sent to every expert."""
    mode = ROUTER_MODES[(score, bool(pre_softmax))]
    if logits.is_cuda and logits.shape[1] <= 256 and k <= 8:
        probs, idx, scores, counts = _RouterTopK.apply(logits.contiguous().float(), bias, k, mode, scaling or 1.0)
        return probs, idx.long(), scores, counts
    if mode == 2:
        scores = torch.sigmoid(logits)
        sel = scores + bias if bias is not None else scores
        idx = sel.topk(k, dim=-1).indices
        probs = scores.gather(1, idx)
        if k > 1:
            probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
    else:
        scores = torch.softmax(logits, dim=-1)
        if mode == 1:
            probs, idx = scores.topk(k, dim=-1)
        else:
            vals, idx = logits.topk(k, dim=-1)
            probs = torch.softmax(vals, dim=-1)
    if scaling:
        probs = probs * scaling
    counts = torch.zeros(logits.shape[1], dtype=torch.float32, device=logits.device)
    counts.index_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=logits.device))
    return probs, idx, scores, counts
