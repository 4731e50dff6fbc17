"""Kernel micro-benchmarks with roofline fractions.

    python -m areal_b200.ops.microbench gemm [--small] [--iters N]
    python -m areal_b200.ops.microbench all

Each benchmark times one op of this library with CUDA events on the launching stream (after
warm-up, synchronised on both sides; an L2-sized buffer is rewritten between iterations unless
the working set already exceeds L2), and prints one JSON line: milliseconds, the algorithmic
FLOP/s or bytes/s, and that figure as a fraction of the measured peaks (``MEASURED_PEAKS.json``
at the repository root when present: cuBLAS bf16 burst throughput and copy bandwidth; otherwise
the documented fall-back figures). ``--small`` shrinks the case to a few hundred MB so that a
profiler capture of one launch finishes quickly.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK, source="fallback")


_FLUSH = None


def timeit(fn, iters: int, warm: int = 3, flush: bool = True) -> float:
    """Mean milliseconds per call."""
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def report(name: str, ms: float, flops: float = 0.0, nbytes: float = 0.0, **extra):
    pk = peaks()
    out = {"op": name, "ms": round(ms, 4)}
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_of_bf16_peak=round(tf / pk["bf16_tflops"], 3))
    if nbytes:
        gbs = nbytes / ms / 1e6
        out.update(gbs=round(gbs, 1), frac_of_hbm_peak=round(gbs / pk["hbm_gbs"], 3))
    out["peaks"] = pk["source"]
    out.update(extra)
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(a):
    from .gemm import gemm

    M, N, K = (2048, 4096, 4096) if a.small else (8192, 8192, 8192)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    ms = timeit(lambda: gemm(x, w), a.iters)
    report("gemm_bf16", ms, flops=2.0 * M * N * K, shape=[M, N, K])
    dy = torch.randn(M, N, device="cuda").bfloat16()
    ms = timeit(lambda: gemm(dy, w, b_mn=True), a.iters)
    report("gemm_bf16_dgrad", ms, flops=2.0 * M * N * K, shape=[M, K, N])
    ms = timeit(lambda: gemm(dy, x, a_mn=True, b_mn=True), a.iters)
    report("gemm_bf16_wgrad", ms, flops=2.0 * M * N * K, shape=[N, K, M])


def bench_gemm_fp8(a):
    from . import fp8

    M, N, K = (2048, 4096, 4096) if a.small else (8192, 8192, 8192)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    a8, sa = fp8.quant_fp8_1x128(x)
    b8, sb = fp8.quant_fp8_block128(w)
    ms = timeit(lambda: fp8.gemm_fp8_block(a8, sa, b8, sb), a.iters)
    report("gemm_fp8_block", ms, flops=2.0 * M * N * K, shape=[M, N, K])
    ms = timeit(lambda: fp8.quant_fp8_1x128(x), a.iters)
    report("quant_fp8_1x128", ms, nbytes=M * K * 3.0)
    ms = timeit(lambda: fp8.quant_fp8_block128(w), a.iters)
    report("quant_fp8_block128", ms, nbytes=N * K * 3.0)


def bench_grouped_gemm(a):
    from . import moe

    T, E, k, H, I = (4096, 32, 4, 2048, 768) if a.small else (16384, 128, 8, 2048, 768)
    x = torch.randn(T, H, device="cuda").bfloat16()
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * H ** -0.5).bfloat16()
    idx, w = moe.route(torch.randn(T, E, device="cuda"), k, True)
    s = moe.sort_by_expert(idx, E)
    xs = moe.gather_rows(x, s)
    ms = timeit(lambda: moe.grouped_gemm(xs, gate_up, s), a.iters)
    report("grouped_gemm_fwd", ms, flops=2.0 * T * k * 2 * I * H, experts=E, rows=T * k)
    dy = torch.randn(s.max_rows, 2 * I, device="cuda").bfloat16()
    ms = timeit(lambda: moe.grouped_wgrad(dy, xs, s), a.iters)
    report("grouped_gemm_wgrad", ms, flops=2.0 * T * k * 2 * I * H, experts=E)
    ms = timeit(lambda: moe.sort_by_expert(idx, E), a.iters)
    report("moe_sort", ms, nbytes=T * k * 12.0)
    ms = timeit(lambda: moe.gather_rows(x, s), a.iters)
    report("moe_gather", ms, nbytes=T * k * H * 2.0 + T * H * 2.0)


def _attn_inputs(a):
    from .attention import VarlenMeta

    nseq, L = (4, 4096) if a.small else (8, 8192)
    Hq, Hkv, D = 16, 8, 128
    T = nseq * L
    q = torch.randn(T, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    meta = VarlenMeta([i * L for i in range(nseq + 1)], "cuda")
    flops = 4.0 * nseq * L * L / 2 * Hq * D
    return q, k, v, meta, flops


def bench_attn(a):
    from .attention import varlen_attention

    q, k, v, meta, flops = _attn_inputs(a)
    with torch.no_grad():
        ms = timeit(lambda: varlen_attention(q, k, v, meta), a.iters)
    report("attn_fwd", ms, flops=flops)
    out = varlen_attention(q, k, v, meta)
    do = torch.randn_like(out)
    ms = timeit(lambda: torch.autograd.grad(out, (q, k, v), do, retain_graph=True), a.iters)
    report("attn_bwd", ms, flops=2.5 * flops)


def bench_lm_head(a):
    from .lm_head import lm_head_logprobs

    T, H, V = (4096, 2048, 151936) if a.small else (16384, 2048, 151936)
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    with torch.no_grad():
        ms = timeit(lambda: lm_head_logprobs(x, w, labels), a.iters)
    report("lm_head_fwd", ms, flops=2.0 * T * H * V)
    lp, ent = lm_head_logprobs(x, w, labels)
    g = torch.randn_like(lp)
    ms = timeit(lambda: torch.autograd.grad(lp, (x, w), g, retain_graph=True), a.iters)
    report("lm_head_bwd", ms, flops=6.0 * T * H * V)  # logits recompute + dx + dw


def bench_decode(a):
    from . import rollout_ops

    B, ctx = (64, 2000) if a.small else (320, 2000)
    Hq, Hkv, D, bs = 16, 8, 128, 16
    nb_per = (ctx + bs - 1) // bs
    nb = B * nb_per
    kc = torch.randn(nb, Hkv, bs, D, device="cuda").bfloat16()
    vc = torch.randn_like(kc)
    bt = torch.randperm(nb, device="cuda").int().view(B, nb_per)
    sl = torch.randint(ctx // 2, ctx + 1, (B,), device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    nbytes = float(sl.sum()) * Hkv * D * 2 * 2
    ms = timeit(lambda: rollout_ops.paged_decode(q, kc, vc, bt, sl, max_seq_len=ctx), a.iters, flush=False)
    report("paged_decode", ms, nbytes=nbytes, batch=B, ctx=ctx)


def bench_elementwise(a):
    from . import fused

    T, H, I = (8192, 2048, 6144) if a.small else (65536, 2048, 6144)
    x = torch.randn(T, H, device="cuda").bfloat16()
    r = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    with torch.no_grad():
        ms = timeit(lambda: fused.rmsnorm(x, w, 1e-6, residual=r), a.iters)
        report("rmsnorm_residual_fwd", ms, nbytes=T * H * 2.0 * 4)
        gu = torch.randn(T, 2 * I, device="cuda").bfloat16()
        ms = timeit(lambda: fused.swiglu(gu), a.iters)
        report("swiglu_fwd", ms, nbytes=T * I * 2.0 * 3)
        del gu
        Hq, Hkv, D = 16, 8, 128
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
        qw, kw = torch.ones(D, device="cuda").bfloat16(), torch.ones(D, device="cuda").bfloat16()
        cos, sin = fused.rope_tables(4096, D, 1e6, "cuda")
        pos = (torch.arange(T, device="cuda") % 4096).int()
        ms = timeit(lambda: fused.qknorm_rope(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, 1e-6), a.iters)
        report("qknorm_rope_fwd", ms, nbytes=T * (Hq + Hkv) * D * 2.0 * 2)


def bench_kchunk_gemm(a):
    """The all-to-all → GEMM kernel's main loop on one GPU: four emulated source ranks whose chunks are
    already in the gather buffer and whose flags already carry the epoch, so the K loop runs its rotated
    chunk order and flag checks without waiting (the exchange itself needs two or more GPUs)."""
    import ctypes

    from . import _lib

    world, rank = 4, 1
    M, Kc, N = (2048, 1024, 4096) if a.small else (8192, 1024, 4096)
    chunks = (torch.randn(world, M, Kc, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(N, world * Kc, device="cuda") * 0.1).bfloat16()
    flags = torch.full((64,), 3, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    lib = _lib.kernels()

    def run():
        rc = lib.b200_gemm_kchunk_gated(_lib.ptr(chunks), _lib.ptr(w), _lib.ptr(out), _lib.ptr(flags), ctypes.c_uint(3),
                                        ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(M), ctypes.c_int(N),
                                        ctypes.c_int(Kc), ctypes.c_longlong(w.stride(0)),
                                        ctypes.c_longlong(out.stride(0)), _lib.stream_ptr())
        _lib.check(rc, "b200_gemm_kchunk_gated")

    ms = timeit(run, a.iters)
    report("gemm_kchunk_gated_emulated", ms, flops=2.0 * M * N * world * Kc, shape=[M, N, world * Kc])


def bench_optimizer(a):
    """Sharded AdamW update (fp32 master + moments in, new bf16 weights out) on one rank's shard."""
    from ..api.cli_args import OptimizerConfig
    from ..engine.flat_params import FlatParams, ShardedAdamW

    n = (1 << 25) if a.small else (1 << 28)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.randn(n, device="cuda").bfloat16())

    for kind, per_elem in (("adam", 4 * 4 + 3 * 4 + 2), ("adam_bf16", 4 + 4 * 2 + 4 * 2)):
        m = M()
        flat = FlatParams(m, "local")
        opt = ShardedAdamW(flat, OptimizerConfig(type=kind, lr=1e-3, gradient_clipping=1.0), total_steps=100)
        opt.shard_grad.normal_()
        opt._norm.fill_(float(n))
        ms = timeit(lambda: opt._update_cuda(), a.iters)
        report(f"optimizer_update_{kind}", ms, nbytes=float(n) * per_elem, numel=n)
        del opt, flat, m
        torch.cuda.empty_cache()


def bench_sampler(a):
    from .rollout_ops import sample

    B, V = (64, 151936) if a.small else (512, 151936)
    logits = torch.randn(B, V, device="cuda")
    temp = torch.ones(B, device="cuda")
    u = torch.rand(B, device="cuda")
    ms = timeit(lambda: sample(logits, temp, None, None, u), a.iters)
    report("sampler", ms, nbytes=B * V * 4.0, batch=B)


def bench_sample_head(a):
    """Decode LM head + sampling at the Qwen3-1.7B head shape: the fused head (token drawn in the GEMM
    epilogue) against GEMM -> fp32 logits -> stand-alone sampler. Roofline: one read of the weight matrix."""
    from .gemm import gemm
    from .lm_head import lm_head_sample, new_sampling_rng
    from .rollout_ops import sample

    H, V = 2048, 151936
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16()
    for B in ((64,) if a.small else (64, 300, 512)):
        x = torch.randn(B, H, device="cuda").bfloat16()
        temp = torch.ones(B, device="cuda")
        u = torch.rand(B, device="cuda")
        rng = new_sampling_rng(1, "cuda")
        nbytes = float(V) * H * 2
        ms = timeit(lambda: lm_head_sample(x, w, temp, rng), a.iters)
        report("lm_head_sample_fused", ms, flops=2.0 * B * V * H, nbytes=nbytes, batch=B)
        ms = timeit(lambda: sample(gemm(x, w, out_dtype=torch.float32), temp, None, None, u), a.iters)
        report("lm_head_gemm_plus_sampler", ms, flops=2.0 * B * V * H, nbytes=nbytes + 2.0 * B * V * 4, batch=B)


def bench_ppo_loss(a):
    from .rl_ops import ppo_loss_fused

    T = (1 << 20) if a.small else (1 << 24)
    mk = lambda: torch.randn(T, device="cuda") * 0.1
    logp, old, prox, adv = mk().requires_grad_(), mk(), mk(), mk()
    mask = (torch.rand(T, device="cuda") > 0.3).float()
    denom = float(mask.sum())
    with torch.no_grad():
        ms = timeit(lambda: ppo_loss_fused(logp, prox, old, adv, mask, eps_clip=0.2, denom=denom), a.iters)
    report("ppo_loss", ms, nbytes=T * 4.0 * 5)


def bench_decode_step(a):
    """One full decode step (all layers, LM head, sampler) of Qwen3-1.7B: eager and as a CUDA graph."""
    import dataclasses

    from ..models.config import PRESETS
    from ..models.qwen import build_model
    from .rollout_ops import sample

    mc = dataclasses.replace(PRESETS["qwen3-1.7b"])
    model = build_model(mc, dtype=torch.bfloat16, device="cuda", seed=0).eval()
    bs = 16
    B, ctx = (64, 1500) if a.small else (256, 1500)
    nb_per = (ctx + bs) // bs + 1
    nb = B * nb_per
    caches = [(torch.zeros(nb, mc.num_key_value_heads, bs, mc.head_dim, dtype=torch.bfloat16, device="cuda"),
               torch.zeros(nb, mc.num_key_value_heads, bs, mc.head_dim, dtype=torch.bfloat16, device="cuda"))
              for _ in range(mc.num_hidden_layers)]
    bt = torch.randperm(nb, device="cuda").int().view(B, nb_per)
    sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    ids = torch.randint(0, 1000, (B,), device="cuda")
    pos = (sl - 1).long()
    slots = bt[:, (ctx - 1) // bs].long() * bs + (ctx - 1) % bs
    temp = torch.ones(B, device="cuda")
    u = torch.rand(B, device="cuda")
    from .lm_head import lm_head_sample, new_sampling_rng

    rng = new_sampling_rng(1, "cuda")

    @torch.no_grad()
    def step():
        h = model.decode(ids, pos, caches, bt, sl, slots, max_seq_len=ctx)
        if getattr(a, "unfused_sampler", False):
            return sample(model.logits(h, out_dtype=torch.float32), temp, None, None, u)
        return lm_head_sample(h, model.output_weight(), temp, rng)

    kv_bytes = float(B) * ctx * mc.num_key_value_heads * mc.head_dim * 2 * 2 * mc.num_hidden_layers
    w_bytes = mc.num_params() * 2.0
    ms = timeit(step, a.iters, flush=False)
    report("decode_step_eager", ms, nbytes=kv_bytes + w_bytes, batch=B, ctx=ctx)
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        step()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=st):
            step()
    torch.cuda.synchronize()
    ms = timeit(g.replay, a.iters, flush=False)
    report("decode_step_graph", ms, nbytes=kv_bytes + w_bytes, batch=B, ctx=ctx, tokens_per_s=round(B / ms * 1e3))


BENCHES = {"gemm": bench_gemm, "gemm_fp8": bench_gemm_fp8, "grouped_gemm": bench_grouped_gemm, "attn": bench_attn,
           "lm_head": bench_lm_head, "decode": bench_decode, "elementwise": bench_elementwise, "optimizer": bench_optimizer, "kchunk_gemm": bench_kchunk_gemm,
           "sampler": bench_sampler, "sample_head": bench_sample_head, "ppo_loss": bench_ppo_loss,
           "decode_step": bench_decode_step}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=sorted(BENCHES) + ["all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--unfused-sampler", action="store_true", help="decode_step: GEMM + logits + stand-alone sampler")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    for name in (sorted(BENCHES) if a.op == "all" else [a.op]):
        BENCHES[name](a)


if __name__ == "__main__":
    main()
