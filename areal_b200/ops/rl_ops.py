"""CUDA entry points for the RL numerics kernels in ``csrc/ppo_loss.cu``:
fused decoupled-PPO loss (value + d loss/d logprob in one pass), group
normalisation of rewards/advantages and the GAE scan over packed sequences.
The PyTorch formulations in ``areal_b200.utils.functional`` are the oracles and
the CPU path.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


class _PPOLossFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, prox, behav, adv, mask, eps_clip, eps_clip_higher, c_clip, behav_cap,
                use_decoupled, denom):
        n = logp.numel()
        logp_c = logp.float().contiguous()
        dlogp = torch.empty_like(logp_c)
        stats = torch.empty(6, dtype=torch.float32, device=logp.device)
        mask_u8 = mask.to(torch.uint8).contiguous()
        lib = _lib.kernels()
        lib.b200_ppo_loss.restype = ctypes.c_int
        rc = lib.b200_ppo_loss(
            _lib.ptr(logp_c), _lib.ptr(prox.float().contiguous()),
            _lib.ptr(behav.float().contiguous()), _lib.ptr(adv.float().contiguous()),
            _lib.ptr(mask_u8), _lib.ptr(dlogp), _lib.ptr(stats), ctypes.c_longlong(n),
            ctypes.c_float(eps_clip),
            ctypes.c_float(-1.0 if eps_clip_higher is None else eps_clip_higher),
            ctypes.c_float(0.0 if c_clip is None else c_clip),
            ctypes.c_float(0.0 if behav_cap is None else behav_cap),
            ctypes.c_float(1.0 / max(float(denom), 1.0)), ctypes.c_int(int(use_decoupled)),
            _lib.stream_ptr())
        _lib.check(rc, "b200_ppo_loss")
        _lib.count_launch()
        ctx.save_for_backward(dlogp)
        ctx.shape = logp.shape
        ctx.mark_non_differentiable(stats)
        return stats[0].clone(), stats

    @staticmethod
    def backward(ctx, g_loss, g_stats):
        (dlogp,) = ctx.saved_tensors
        return (dlogp * g_loss).view(ctx.shape), None, None, None, None, None, None, None, None, None, None


def ppo_loss_fused(logp, prox, behav, adv, mask, *, eps_clip, eps_clip_higher=None, c_clip=None,
                   behav_cap=None, use_decoupled=True, behav_weight=None, denom=None):
    """Token-level decoupled PPO loss. Returns ``(loss, stats[6])`` where stats =
    [loss, #clipped, #dual-clipped, sum importance weight, sum |ratio-1|, #dropped].

    ``use_decoupled``: the ratio is taken against ``prox`` (else against ``behav``). ``behav_weight``: the
    loss is also multiplied by ``exp(prox - behav)``, dropped above ``behav_cap`` — what token-level
    ratio rejection sampling with action ``mask`` does; the default applies it exactly when a cap is given
    (without rejection sampling the reference's loss carries no such weight:
    areal/utils/functional/functional.py:429-559)."""
    if denom is None:
        denom = mask.count_nonzero()
    if behav_weight is None:
        behav_weight = behav_cap is not None
    flags = int(bool(use_decoupled)) | (2 if behav_weight else 0)
    return _PPOLossFused.apply(logp, prox, behav, adv, mask, eps_clip, eps_clip_higher, c_clip,
                               behav_cap, flags, float(denom))


def group_norm(values: torch.Tensor, group_size: int, *, mean_group=True, std_group=True,
               leave1out=False, unbiased=True, eps=1e-5) -> torch.Tensor:
    """Normalises ``values [n_groups * group_size]`` inside consecutive groups."""
    assert values.numel() % group_size == 0
    v = values.float().contiguous()
    out = torch.empty_like(v)
    lib = _lib.kernels()
    lib.b200_group_norm.restype = ctypes.c_int
    rc = lib.b200_group_norm(_lib.ptr(v), _lib.ptr(out), ctypes.c_int(v.numel() // group_size),
                             ctypes.c_int(group_size), ctypes.c_int(int(mean_group)),
                             ctypes.c_int(int(std_group)), ctypes.c_int(int(leave1out)),
                             ctypes.c_int(int(unbiased)), ctypes.c_float(eps), _lib.stream_ptr())
    _lib.check(rc, "b200_group_norm")
    _lib.count_launch()
    return out.view(values.shape)


def gae_packed(rewards, values, loss_mask, cu_seqlens, no_eos, gamma: float, lam: float):
    """GAE over packed sequences; returns ``(advantages, returns)``."""
    r = rewards.float().contiguous()
    adv = torch.empty_like(r)
    ret = torch.empty_like(r)
    vals = values.float().contiguous() if values is not None else None
    ne = no_eos.to(torch.uint8).contiguous() if no_eos is not None else None
    lib = _lib.kernels()
    lib.b200_gae.restype = ctypes.c_int
    rc = lib.b200_gae(_lib.ptr(r), _lib.ptr(vals), _lib.ptr(loss_mask.to(torch.uint8).contiguous()),
                      _lib.ptr(cu_seqlens.to(torch.int32).contiguous()), _lib.ptr(ne),
                      _lib.ptr(adv), _lib.ptr(ret), ctypes.c_int(cu_seqlens.numel() - 1),
                      ctypes.c_float(gamma), ctypes.c_float(lam), _lib.stream_ptr())
    _lib.check(rc, "b200_gae")
    _lib.count_launch()
    return adv, ret
