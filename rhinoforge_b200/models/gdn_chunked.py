"""Gated delta rule: the token-by-token recurrence and its chunked (block-parallel) form, in plain PyTorch.

The device path (``csrc/kernels/gdn.cu``) runs the recurrence; this module is the host-side statement of both forms -
the oracle of the kernel tests and the algorithm a chunked prefill kernel has to implement (the reference runs prefill in
64-token chunks: ``src/fused/rpu_qwen3_5_model.h:1-20,88-110``, helper operators ``rpu_cumsum.cpp``,
``rpu_unit_tril_inv.cpp``).

Per head, with state ``S [Dk, Dv]``, log-decay ``g_t <= 0`` and write strength ``beta_t``::

    S  <- exp(g_t) * S
    u_t = beta_t * (v_t - k_t^T S)            # what the state does not yet predict
    S  <- S + k_t (x) u_t
    o_t = q_t^T S

Inside a chunk of C tokens with incoming state ``S0`` and cumulative decay ``G_i = sum_{j<=i} g_j`` this unrolls to a
unit-lower-triangular system::

    (I + L) U = beta*V - (beta * e^G * K) S0,      L_ij = beta_i e^{G_i - G_j} (k_i . k_j)  for j < i
    O  = (e^G * Q) S0 + tril(e^{G_i - G_j} (q_i . k_j)) U
    S' = e^{G_C} S0 + (e^{G_C - G} * K)^T U

so a chunk costs a handful of C x C and C x D matrix products plus one triangular inverse (``(I + L)^{-1}``, what
``rf_unit_tril_inv_f32`` computes) instead of C dependent steps.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def recurrent_gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                               state: Optional[torch.Tensor] = None, scale: Optional[float] = None
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q, k [T, H, Dk]``, ``v [T, H, Dv]``, ``g, beta [T, H]`` -> ``(o [T, H, Dv], state [H, Dk, Dv])`` in fp32."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    S = torch.zeros(H, Dk, Dv) if state is None else state.float().clone()
    S = S.to(q.device)
    out = torch.empty(T, H, Dv, device=q.device)
    for t in range(T):
        S = S * torch.exp(g[t])[:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hk,hkv->hv", k[t], S))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hk,hkv->hv", q[t] * scale, S)
    return out, S


def chunked_gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                             state: Optional[torch.Tensor] = None, scale: Optional[float] = None, chunk: int = 64
                             ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as :func:`recurrent_gated_delta_rule`, evaluated chunk by chunk (any ``T``; the last chunk may be
    short)."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    dev = q.device
    q, k, v, g, beta = (t.float().transpose(0, 1) for t in (q * 1.0, k, v, g, beta))     # head-major: [H, T, ...]
    q = q * scale
    S = (torch.zeros(H, Dk, Dv) if state is None else state.float().clone()).to(dev)
    out = torch.empty(H, T, Dv, device=dev)
    for c0 in range(0, T, chunk):
        sl = slice(c0, min(c0 + chunk, T))
        qc, kc, vc, gc, bc = q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl]
        C = qc.shape[1]
        G = torch.cumsum(gc, dim=1)                                           # [H, C]
        decay = torch.exp(G[:, :, None] - G[:, None, :])                      # e^{G_i - G_j}
        lower = torch.tril(torch.ones(C, C, device=dev), -1)
        L = bc[:, :, None] * decay * torch.einsum("hik,hjk->hij", kc, kc) * lower
        eye = torch.eye(C, device=dev).expand(H, C, C)
        rhs = bc[:, :, None] * vc - torch.einsum("hck,hkv->hcv", bc[:, :, None] * torch.exp(G)[:, :, None] * kc, S)
        U = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
        qk = torch.einsum("hik,hjk->hij", qc, kc) * decay * torch.tril(torch.ones(C, C, device=dev))
        out[:, sl] = torch.einsum("hck,hkv->hcv", torch.exp(G)[:, :, None] * qc, S) + torch.einsum("hij,hjv->hiv", qk, U)
        tail = torch.exp(G[:, -1:, None] - G[:, :, None])                     # e^{G_C - G_j}
        S = torch.exp(G[:, -1])[:, None, None] * S + torch.einsum("hck,hcv->hkv", tail * kc, U)
    return out.transpose(0, 1).contiguous(), S


__all__ = ["recurrent_gated_delta_rule", "chunked_gated_delta_rule"]
