"""Rollout-engine ops: paged KV-cache write, paged decode attention and fused
sampling (``csrc/paged_decode.cu``, ``csrc/sampler.cu``) with PyTorch references."""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib


def kv_cache_write(k, v, slot_mapping, k_cache, v_cache):
    """Writes ``k, v [T, Hkv, D]`` (token pitch may be larger) into the paged caches
    ``[num_blocks, Hkv, block_size, D]`` at flat slots ``slot_mapping [T]`` (int64,
    ``block * block_size + offset``; negative slots are skipped)."""
    T, Hkv, D = k.shape
    bs = k_cache.shape[2]
    if not (_lib.use_cuda_kernels(k, v, k_cache) and D == 128):  # the kernel is written for head_dim 128
        ok = slot_mapping >= 0
        sm = slot_mapping[ok].long()
        blk, off = sm // bs, sm % bs
        k_cache[blk, :, off] = k[ok].to(k_cache.dtype)
        v_cache[blk, :, off] = v[ok].to(v_cache.dtype)
        return
    if _lib.checked():
        _lib.check_operand("kv_cache_write.k_cache", k_cache, None, (None, Hkv, bs, D))
        _lib.check_operand("kv_cache_write.v_cache", v_cache, None, tuple(k_cache.shape))
        _lib.check_index("kv_cache_write.slot_mapping", slot_mapping[:T], k_cache.shape[0] * bs, allow_negative=True)
    lib = _lib.kernels()
    lib.b200_kv_cache_write.restype = ctypes.c_int
    rc = lib.b200_kv_cache_write(_lib.ptr(k), _lib.ptr(v), ctypes.c_longlong(k.stride(0)),
                                 ctypes.c_longlong(v.stride(0)),
                                 _lib.ptr(slot_mapping.to(torch.int64).contiguous()),
                                 _lib.ptr(k_cache), _lib.ptr(v_cache), ctypes.c_int(T),
                                 ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(bs), _lib.stream_ptr())
    _lib.check(rc, "b200_kv_cache_write")
    _lib.count_launch()


def paged_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale=None):
    B, Hq, D = q.shape
    nb, Hkv, bs, _ = k_cache.shape
    scale = scale or 1.0 / math.sqrt(D)
    g = Hq // Hkv
    out = torch.zeros((B, Hq, D), dtype=torch.float32, device=q.device)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        blocks = block_table[b, : (L + bs - 1) // bs].long()
        k = k_cache[blocks].transpose(1, 2).reshape(-1, Hkv, D)[:L].float().repeat_interleave(g, 1)
        v = v_cache[blocks].transpose(1, 2).reshape(-1, Hkv, D)[:L].float().repeat_interleave(g, 1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), k) * scale
        out[b] = torch.einsum("hl,lhd->hd", s.softmax(-1), v)
    return out.to(q.dtype)


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale=None, nsplit: int | None = None,
                 max_seq_len: int | None = None):
    """One query token per sequence attending to its paged cache (GQA)."""
    B, Hq, D = q.shape
    scale = scale or 1.0 / math.sqrt(D)
    nb, Hkv, bs, _ = k_cache.shape
    if not (_lib.use_cuda_kernels(q, k_cache) and q.dtype == torch.bfloat16 and D == 128 and bs % 16 == 0):
        return paged_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale)
    if nsplit is None:
        # enough CTAs to fill the GPU (two resident per SM); long sequences get more splits
        ctas = B * Hkv
        nsplit = 1
        if max_seq_len is None:
            max_seq_len = block_table.shape[1] * bs
        while ctas * nsplit < 592 and nsplit < 32 and max_seq_len // (nsplit * 2) >= 256:
            nsplit *= 2
    q = q if q.is_contiguous() else q.contiguous()
    out = torch.empty_like(q)
    if nsplit > 1:
        o_part = torch.empty((B, Hq, nsplit, D), dtype=torch.float32, device=q.device)
        ml_part = torch.empty((B, Hq, nsplit, 2), dtype=torch.float32, device=q.device)
    else:
        o_part = ml_part = None
    if _lib.checked():
        max_blocks = block_table.shape[1]
        _lib.check_operand("paged_decode.block_table", block_table, torch.int32, (None, max_blocks), align=4)
        _lib.check_operand("paged_decode.seq_lens", seq_lens, torch.int32, None, align=4)
        _lib.check_operand("paged_decode.k_cache", k_cache, torch.bfloat16, (nb, Hkv, bs, D))
        _lib.check_operand("paged_decode.v_cache", v_cache, torch.bfloat16, (nb, Hkv, bs, D))
        lens = seq_lens[:B].long()
        _lib.check_index("paged_decode.seq_lens", lens, max_blocks * bs + 1)
        used = torch.arange(max_blocks, device=q.device)[None, :] < ((lens + bs - 1) // bs)[:, None]
        _lib.check_index("paged_decode.block_table", block_table[:B], nb, where=used)
    lib = _lib.kernels()
    lib.b200_paged_decode.restype = ctypes.c_int
    rc = lib.b200_paged_decode(_lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache),
                               _lib.ptr(block_table), _lib.ptr(seq_lens), _lib.ptr(out),
                               _lib.ptr(o_part), _lib.ptr(ml_part), ctypes.c_int(B),
                               ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D),
                               ctypes.c_int(bs), ctypes.c_int(nb), ctypes.c_int(block_table.shape[1]),
                               ctypes.c_int(nsplit), ctypes.c_float(scale), _lib.stream_ptr())
    _lib.check(rc, "b200_paged_decode")
    _lib.count_launch(2 if nsplit > 1 else 1)
    return out


def sample_ref(logits, temperature, top_k, top_p, uniforms):
    """Inverse-CDF sampling in PyTorch with the same conventions as the kernel."""
    B, V = logits.shape
    tokens = torch.empty(B, dtype=torch.int32, device=logits.device)
    logps = torch.empty(B, dtype=torch.float32, device=logits.device)
    for b in range(B):
        t = float(temperature[b])
        x = logits[b].float()
        if t <= 0:
            tok = int(x.argmax())
            tokens[b] = tok
            logps[b] = torch.log_softmax(x, -1)[tok]
            continue
        y = x / t
        lsm = torch.log_softmax(y, -1)
        p = lsm.exp()
        keep = torch.ones(V, dtype=torch.bool, device=logits.device)
        k = int(top_k[b]) if top_k is not None else 0
        if 0 < k < V:
            kth = torch.topk(p, k).values[-1]
            keep &= p >= kth
        pp = float(top_p[b]) if top_p is not None else 1.0
        if pp < 1.0:
            sp, si = torch.sort(p, descending=True)
            cum = sp.cumsum(0)
            n_keep = int((cum < pp).sum()) + 1
            thr = sp[min(n_keep, V) - 1]
            keep &= p >= thr
        pk = torch.where(keep, p, torch.zeros_like(p))
        cdf = pk.double().cumsum(0)
        target = float(uniforms[b]) * float(cdf[-1])
        tok = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64,
                                                       device=logits.device), right=True))
        tok = min(tok, V - 1)
        tokens[b] = tok
        logps[b] = lsm[tok]
    return tokens, logps


def sample(logits, temperature, top_k=None, top_p=None, uniforms=None, generator=None):
    """Draws one token per row of fp32 ``logits [B, V]``; returns ``(tokens int32, logprobs f32)``.
    ``temperature[b] <= 0`` means greedy."""
    B, V = logits.shape
    if uniforms is None:
        uniforms = torch.rand(B, device=logits.device, generator=generator, dtype=torch.float32)
    if not _lib.use_cuda_kernels(logits):
        return sample_ref(logits, temperature, top_k, top_p, uniforms)
    logits = logits.float()
    logits = logits if logits.stride(1) == 1 else logits.contiguous()
    tokens = torch.empty(B, dtype=torch.int32, device=logits.device)
    logps = torch.empty(B, dtype=torch.float32, device=logits.device)
    lib = _lib.kernels()
    lib.b200_sample.restype = ctypes.c_int
    rc = lib.b200_sample(_lib.ptr(logits), ctypes.c_longlong(logits.stride(0)), ctypes.c_int(B),
                         ctypes.c_int(V), _lib.ptr(temperature.float().contiguous()),
                         _lib.ptr(top_k.to(torch.int32).contiguous()) if top_k is not None else None,
                         _lib.ptr(top_p.float().contiguous()) if top_p is not None else None,
                         _lib.ptr(uniforms.float().contiguous()), _lib.ptr(tokens), _lib.ptr(logps),
                         _lib.stream_ptr())
    _lib.check(rc, "b200_sample")
    _lib.count_launch()
    return tokens, logps
