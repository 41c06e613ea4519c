"""Sparse mixture-of-experts MLP (LingBot-VLA-v2 expert geometry: sigmoid router with correction bias,
top-4 of 32, normalised top-k weights times a routed scaling factor, plus an always-on shared expert).

Two execution forms over ONE packed expert bank (gates and ups of all experts stacked along N, downs
concatenated along K; the always-on shared expert occupies the trailing columns):

* dense einsum (up to ``dense_max_tokens`` rows): every expert's gate/up projection is one column block of a
  single GEMM, the routing weight (zero when the expert was not selected) scales the block, and the down
  projections form one GEMM over ``K = E * I (+ I_shared)`` that sums the weighted expert outputs.  With a
  few dozen tokens every expert is picked by someone, so both forms read every expert's weights once and this
  one needs the fewest launches;
* grouped GEMM (more rows): the picks are bucketed by expert, their rows gathered in that order, and one
  persistent launch per projection multiplies each expert's rows with that expert's weights only
  (``top_k / E`` of the dense form's FLOPs); the shared expert runs as an ordinary GLU MLP and a combine step
  adds every token's picks in pick order.

Tensor parallelism shards ``I`` of every expert over the ranks (no expert parallelism, no all-to-all), as in
the reference (``src/fused/rpu_lingbot_v2_moe_model.h:29-49``, ``.cpp:1029-1213,1215-1312,1317-1511``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch
import torch.nn.functional as F

from ..ops import kernels as K


@dataclass
class MoEConfig:
    hidden: int
    experts: int = 32
    top_k: int = 4
    expert_inter: int = 512
    shared_inter: int = 0              # 0: no shared expert
    routed_scale: float = 4.0
    norm_topk: bool = True
    score_fn: str = "sigmoid"


class MoEMLP:
    """``forward(x [T, hidden]) -> [T, hidden]`` (no residual).  Weights: ``router.weight [E, H]``,
    ``router.bias [E]`` (the selection-only correction bias, optional), ``experts.{e}.{gate,up,down}_proj.weight``,
    ``shared.{gate,up,down}_proj.weight`` (optional)."""

    def __init__(self, cfg: MoEConfig, sd: Dict[str, torch.Tensor], *, prefix: str = "", device="cuda",
                 dtype=torch.float16, tp_rank: int = 0, tp_world: int = 1, dense_max_tokens: int = 256):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.dense_max_tokens = dense_max_tokens
        E, I = cfg.experts, cfg.expert_inter
        if I % tp_world or cfg.shared_inter % tp_world:
            raise ValueError("expert widths must split over the tensor-parallel ranks")
        Il, Sl = I // tp_world, cfg.shared_inter // tp_world
        sl = slice(tp_rank * Il, (tp_rank + 1) * Il)
        ss = slice(tp_rank * Sl, (tp_rank + 1) * Sl)
        g = lambda n: sd[prefix + n]
        dev = lambda t: t.to(self.device, dtype).contiguous()
        gates = [g(f"experts.{e}.gate_proj.weight")[sl] for e in range(E)]
        ups = [g(f"experts.{e}.up_proj.weight")[sl] for e in range(E)]
        downs = [g(f"experts.{e}.down_proj.weight")[:, sl] for e in range(E)]
        if Sl:
            gates.append(g("shared.gate_proj.weight")[ss]); ups.append(g("shared.up_proj.weight")[ss])
            downs.append(g("shared.down_proj.weight")[:, ss])
        self.w_gate_up = dev(torch.cat(gates + ups, 0))            # [2 * (E*Il + Sl), H]: gates then ups
        self.w_down = dev(torch.cat(downs, 1))                     # [H, E*Il + Sl]
        self.router_w = dev(g("router.weight"))
        b = sd.get(prefix + "router.bias")
        self.router_b = None if b is None else b.to(self.device, torch.float32).contiguous()
        self.local_inter, self.local_shared = Il, Sl
        self._packed = None

    def _bank(self):
        """Tile-major images of the bank for the grouped form (built on first use; the experts' row tiles and k blocks
        are addressed inside them, so neither is a per-expert copy)."""
        if self._packed is None:
            self._packed = (K.pack_weight(self.w_gate_up, 2), K.pack_weight(self.w_down))
        return self._packed

    def forward_grouped(self, x: torch.Tensor, *, status=None) -> torch.Tensor:
        cfg, Il, Sl, E = self.cfg, self.local_inter, self.local_shared, self.cfg.experts
        if Il % 128:
            raise ValueError(f"the grouped form needs the local expert width ({Il}) to be a multiple of 128")
        H = cfg.hidden
        pgu, pdn = self._bank()
        logits = K.gemm(x, self.router_w)
        ids, w = K.moe_select(logits, cfg.top_k, bias=self.router_b, score_fn=cfg.score_fn, norm_topk=cfg.norm_topk,
                              scale=cfg.routed_scale)
        slot_of, token_of_slot, slot_w, tiles = K.moe_group(ids, w, E)
        xg = torch.empty((x.shape[0] * cfg.top_k, H), dtype=x.dtype, device=x.device)
        K.embedding(x, token_of_slot, out=xg)                               # row gather in expert order
        bank_rows, bank_k = E * Il + Sl, E * Il + Sl
        hg = K.moe_grouped_gemm(xg, pgu, tiles, n=Il, k=H, bank_rows=bank_rows, bank_k=H, expert_rows=Il, dual=True,
                                act="silu_mul", status=status)
        yg = K.moe_grouped_gemm(hg, pdn, tiles, n=H, k=Il, bank_rows=H, bank_k=bank_k, expert_k=Il, row_scale=slot_w,
                                status=status)
        if Sl:
            gs = self.w_gate_up[E * Il:E * Il + Sl]
            us = self.w_gate_up[bank_rows + E * Il:bank_rows + E * Il + Sl]
            hs = K.gemm(x, torch.cat((gs, us), 0).contiguous(), act="silu_mul", dual=True)
            out = K.gemm(hs, self.w_down[:, E * Il:].contiguous())
        else:
            out = torch.zeros((x.shape[0], H), dtype=x.dtype, device=x.device)
        return K.moe_combine(out, yg, slot_of, cfg.top_k)

    def forward(self, x: torch.Tensor, *, comm=None) -> torch.Tensor:
        cfg = self.cfg
        if x.shape[0] > self.dense_max_tokens and comm is None and self.local_inter % 128 == 0:
            return self.forward_grouped(x)
        logits = K.gemm(x, self.router_w)
        _, _, dense = K.moe_select(logits, cfg.top_k, bias=self.router_b, score_fn=cfg.score_fn,
                                   norm_topk=cfg.norm_topk, scale=cfg.routed_scale, dense=True)
        h = K.gemm(x, self.w_gate_up, act="silu_mul", dual=True)
        K.moe_scale_blocks(h, dense, cfg.experts, self.local_inter)
        return K.gemm(h, self.w_down, comm=comm)

    __call__ = forward


def moe_reference(cfg: MoEConfig, sd: Dict[str, torch.Tensor], x: torch.Tensor, prefix: str = "") -> torch.Tensor:
    """Token-by-token sparse evaluation in fp32 (what the dense-einsum form must equal)."""
    g = lambda n: sd[prefix + n].float()
    xf = x.float()
    logits = (xf @ g("router.weight").t()).to(x.dtype).float()       # the router GEMM stores 16-bit logits
    sc = torch.sigmoid(logits) if cfg.score_fn == "sigmoid" else torch.softmax(logits, -1)
    key = sc + (sd[prefix + "router.bias"].float() if prefix + "router.bias" in sd else 0.0)
    top = torch.topk(key, cfg.top_k, dim=-1).indices
    w = torch.gather(sc, 1, top)
    if cfg.norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * cfg.routed_scale
    out = torch.zeros(x.shape[0], cfg.hidden, dtype=torch.float32, device=x.device)
    mlp = lambda p, t: (F.silu(t @ g(p + "gate_proj.weight").t()) * (t @ g(p + "up_proj.weight").t())) @ g(p + "down_proj.weight").t()
    for t in range(x.shape[0]):
        for j in range(cfg.top_k):
            out[t] += w[t, j] * mlp(f"experts.{int(top[t, j])}.", xf[t:t + 1])[0]
    if cfg.shared_inter:
        out += mlp("shared.", xf)
    return out
