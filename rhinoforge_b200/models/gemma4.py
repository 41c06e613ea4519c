"""Gemma4 text decoder: mixed layer geometry (sliding-window layers with heads of 256, global layers with heads of 512
and proportional RoPE), four RMSNorms per block, per-head q / k norms, an unweighted value norm, attention without a
score scale, K/V shared by the last layers with an earlier layer of their type, per-layer embeddings and a per-layer
output scalar.

One block (``norm`` is RMSNorm with its weight used directly)::

    a = attn(norm_in(h))                 # q, k: per-head norm then RoPE; v: unweighted per-head norm; scale 1
    h = h + norm_post_attn(a Wo)
    h = h + norm_post_ff(Wd (gelu_tanh(Wg f) * (Wu f))),  f = norm_pre_ff(h)
    h = h + norm_post_ple(Wp (gelu_tanh(Wpg h) * e_l))     # e_l: this layer's slice of the per-layer embeddings
    h = h * layer_scalar

The layers are composed from the library's kernels (tcgen05 GEMMs with the GeGLU / activation epilogues, RMSNorm,
the fused per-head norm + rotary + value-norm kernel, the tcgen05 attention for heads of 256 with its sliding-window
mask, the wide-head attention kernel for heads of 512); K and V live in contiguous per-layer buffers, one per layer
that owns its K/V - a sharing layer projects only its queries and reads its donor's buffer.  Rows of a batch are packed
(variable lengths); a decode step is the same path with one row per sequence and replays from a CUDA graph.

Reference behaviour: ``src/fused/rpu_gemma4_model.cpp:1-24,57-90`` (geometry, norms, scale 1, NeoX rotary with half-width
tables, v_norm, KV sharing, PLE, layer scalar), ``python/rpu_backend/adapters/gemma4/geometry.py`` (layer table).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..adapters.gemma4.geometry import LayerGeom, layer_geometry
from ..runtime.errors import RPUBackendError, UnsupportedModelError


def _g(cfg, key, default=None):
    return cfg.get(key, default) if isinstance(cfg, dict) else getattr(cfg, key, default)


def rope_tables(text_config, layer_type: str, head_dim: int, max_pos: int):
    """``(cos, sin) [max_pos, head_dim / 2]`` fp32 for one layer type: plain RoPE on the sliding layers; on the global
    layers only the first ``partial_rotary_factor`` of the frequencies rotate, the rest keep angle zero."""
    rp = _g(text_config, "rope_parameters")[layer_type]
    base, kind = float(rp["rope_theta"]), rp.get("rope_type", "default")
    half = head_dim // 2
    if kind == "proportional":
        rot = int(float(rp.get("partial_rotary_factor", 1.0)) * head_dim // 2)
        inv = torch.zeros(half, dtype=torch.float64)
        inv[:rot] = 1.0 / base ** (torch.arange(0, 2 * rot, 2, dtype=torch.float64) / head_dim)
        inv = inv / float(rp.get("factor", 1.0))
    elif kind == "default":
        inv = 1.0 / base ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim)
    else:
        raise UnsupportedModelError(f"Gemma4 rope_type {kind!r} on {layer_type} layers is not built")
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None].double()
    return ang.cos().float(), ang.sin().float()


def preflight(text_config) -> List[LayerGeom]:
    geo = layer_geometry(text_config)
    bad = []
    if _g(text_config, "enable_moe_block", False):
        bad.append("the mixture-of-experts block")
    if _g(text_config, "hidden_activation", "gelu_pytorch_tanh") != "gelu_pytorch_tanh":
        bad.append(f"activation {_g(text_config, 'hidden_activation')!r}")
    if _g(text_config, "use_bidirectional_attention", None) not in (None, False):
        bad.append("bidirectional attention")
    for g in geo:
        if g.head_dim not in (64, 128, 256, 512):
            bad.append(f"head_dim {g.head_dim} on layer {g.idx}")
            break
    if _g(text_config, "hidden_size") % 8 or _g(text_config, "intermediate_size") % 8:
        bad.append("widths that are not multiples of 8")
    if bad:
        raise UnsupportedModelError("Gemma4 configuration is outside what this framework runs: " + "; ".join(bad))
    return geo


class Gemma4Engine:
    def __init__(self, text_config, get_weight: Callable[[str], torch.Tensor], *, prefix: str = "model.", max_seq_len: int = 2048,
                 max_batch: int = 1, max_tokens: int = 2048, device="cuda", dtype=torch.bfloat16):
        from ..ops import kernels as K
        self.K, self.cfg, self.device, self.dtype = K, text_config, torch.device(device), dtype
        self.geo = preflight(text_config)
        c, dev = text_config, self.device
        self.H, self.L = int(_g(c, "hidden_size")), int(_g(c, "num_hidden_layers"))
        self.inter, self.eps = int(_g(c, "intermediate_size")), float(_g(c, "rms_norm_eps", 1e-6))
        self.P = int(_g(c, "hidden_size_per_layer_input", 0) or 0)
        self.vocab = int(_g(c, "vocab_size"))
        self.softcap = _g(c, "final_logit_softcapping", None)
        self.S, self.B, self.T = max_seq_len, max_batch, max_tokens
        owners_end = self.L - int(_g(c, "num_kv_shared_layers", 0) or 0)
        double_wide = bool(_g(c, "use_double_wide_mlp", False))
        t = lambda w: w.to(dev, dtype).contiguous()
        pack = lambda w: K.pack_weight(t(w))
        get = lambda n: get_weight(prefix + n)
        self.embed = t(get("embed_tokens.weight"))
        try:
            self.lm_head = t(get_weight("lm_head.weight"))
        except KeyError:
            self.lm_head = self.embed                                   # tied
        self.final_w = t(get("norm.weight"))
        if self.P:
            self.ple_embed = t(get("embed_tokens_per_layer.weight"))    # [vocab_ple, L * P]
            self.ple_proj_w = pack(get("per_layer_model_projection.weight").float() * (self.H ** -0.5))
            self.ple_norm_w = t(get("per_layer_projection_norm.weight"))
        self.tables = {}
        for g in self.geo:
            if g.layer_type not in self.tables:
                cos, sin = rope_tables(c, g.layer_type, g.head_dim, max_seq_len)
                self.tables[g.layer_type] = (cos.to(dev), sin.to(dev))
        self.layers = []
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        for g in self.geo:
            p = f"layers.{g.idx}."
            hd, Hq, Hkv = g.head_dim, g.num_q_heads, g.num_kv_heads
            Lw = {"geo": g}
            q = get(p + "self_attn.q_proj.weight")
            if g.has_kv_proj:
                k = get(p + "self_attn.k_proj.weight")
                try:
                    v = get(p + "self_attn.v_proj.weight")
                except KeyError:
                    v = k                                               # keys double as values on this layer
                Lw["qkv_w"], Lw["qkv_rows"] = pack(torch.cat((q, k, v), 0)), (Hq + 2 * Hkv) * hd
                Lw["k_norm"] = t(get(p + "self_attn.k_norm.weight"))
                self.k_cache[g.idx] = torch.zeros(max_batch * max_seq_len, Hkv * hd, dtype=dtype, device=dev)
                self.v_cache[g.idx] = torch.zeros(max_batch * max_seq_len, Hkv * hd, dtype=dtype, device=dev)
            else:
                Lw["qkv_w"], Lw["qkv_rows"] = pack(q), Hq * hd
                Lw["k_norm"] = None
            Lw["q_norm"] = t(get(p + "self_attn.q_norm.weight"))
            Lw["o_w"] = pack(get(p + "self_attn.o_proj.weight"))
            inter = self.inter * (2 if (double_wide and g.idx >= owners_end > 0) else 1)
            Lw["inter"] = inter
            Lw["gu_w"] = K.pack_weight(t(torch.cat((get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")), 0)), sections=2)
            Lw["down_w"] = pack(get(p + "mlp.down_proj.weight"))
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                Lw[n] = t(get(p + n + ".weight"))
            if self.P:
                Lw["ple_gate_w"] = pack(get(p + "per_layer_input_gate.weight"))
                Lw["ple_proj_w"] = pack(get(p + "per_layer_projection.weight"))
                Lw["ple_norm"] = t(get(p + "post_per_layer_input_norm.weight"))
            try:
                Lw["scalar"] = float(get(p + "layer_scalar").reshape(-1)[0])
            except KeyError:
                Lw["scalar"] = 1.0
            self.layers.append(Lw)
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=dev)
        T = max_tokens
        wide = max(L_["qkv_rows"] for L_ in self.layers)
        att_w = max(g.num_q_heads * g.head_dim for g in self.geo)
        self.h, self.n, self.tmp, self.o = z(T, self.H), z(T, self.H), z(T, self.H), z(T, self.H)
        self.qkv, self.att = z(T, wide), z(T, att_w)
        self.ff = z(T, max(L_["inter"] for L_ in self.layers))
        if self.P:
            self.ple, self.ple_in, self.ple_g = z(T, self.L * self.P), z(T, self.L * self.P), z(T, self.P)
        self.lengths = [0] * max_batch
        self.status = torch.zeros(32, dtype=torch.int32, device=dev)
        # decode state (device side, advanced inside the graph)
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        self.d_ids, self.d_pos, self.d_kvlen, self.d_rows = i32(max_batch), i32(max_batch), i32(max_batch), i32(max_batch)
        self.d_qstart = torch.arange(max_batch, dtype=torch.int32, device=dev)
        self.d_qlen = torch.ones(max_batch, dtype=torch.int32, device=dev)
        self.d_kvstart = torch.arange(max_batch, dtype=torch.int32, device=dev) * max_seq_len
        self.d_next = i32(max_batch)
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}

    # ------------------------------------------------------------------------------------------------------------------
    def reset(self) -> None:
        self.lengths = [0] * self.B

    def _run(self, T: int, ids, pos, rows, q_start, q_len, kv_start, kv_len, max_q_len: int) -> None:
        """The decoder over ``T`` packed rows; all index arguments are int32 device tensors."""
        K, H, eps = self.K, self.H, self.eps
        h, n, tmp, o = self.h[:T], self.n[:T], self.tmp[:T], self.o[:T]
        K.embedding(self.embed, ids, out=h, scale=math.sqrt(H))
        if self.P:
            P, L = self.P, self.L
            ple, ple_in = self.ple[:T], self.ple_in[:T]
            K.embedding(self.ple_embed, ids, out=ple_in, scale=math.sqrt(P))
            K.gemm(h, self.ple_proj_w, packed_shape=(L * P, H), out=ple)
            K.rmsnorm(ple.view(T * L, P), self.ple_norm_w, eps, out=ple.view(T * L, P))
            ple.add_(ple_in).mul_(2.0 ** -0.5)
        for Lw in self.layers:
            g: LayerGeom = Lw["geo"]
            hd, Hq, Hkv = g.head_dim, g.num_q_heads, g.num_kv_heads
            cos, sin = self.tables[g.layer_type]
            qkv = self.qkv[:T, :Lw["qkv_rows"]]
            K.rmsnorm(h, Lw["input_layernorm"], eps, out=n)
            K.gemm(n, Lw["qkv_w"], packed_shape=(Lw["qkv_rows"], H), out=qkv)
            own = g.has_kv_proj
            K.qk_norm_rope_kv(qkv, Hq, Hkv if own else 0, hd, pos=pos, cos=cos, sin=sin, rot_dim=hd, q_norm_w=Lw["q_norm"],
                              k_norm_w=Lw["k_norm"], eps=eps, write_k_inplace=True, v_norm=own)
            if own:
                K.scatter_rows(self.k_cache[g.idx], qkv[:, Hq * hd:(Hq + Hkv) * hd], rows)
                K.scatter_rows(self.v_cache[g.idx], qkv[:, (Hq + Hkv) * hd:], rows)
            src = g.kv_source_layer
            att = self.att[:T, :Hq * hd]
            K.attention_prefill(qkv[:, :Hq * hd], att, Hq=Hq, Hkv=Hkv, hd=hd, q_start=q_start, q_len=q_len, kv_len=kv_len,
                                max_q_len=max_q_len, k=self.k_cache[src], v=self.v_cache[src], kv_start=kv_start, causal=True,
                                window=int(g.sliding_window or 0), scale=1.0, status=self.status)
            K.gemm(att, Lw["o_w"], packed_shape=(H, Hq * hd), out=o)
            K.rmsnorm(o, Lw["post_attention_layernorm"], eps, out=tmp)
            h.add_(tmp)
            K.rmsnorm(h, Lw["pre_feedforward_layernorm"], eps, out=n)
            ff = self.ff[:T, :Lw["inter"]]
            K.gemm(n, Lw["gu_w"], packed_shape=(2 * Lw["inter"], H), dual=True, act="gelu_tanh_mul", out=ff)
            K.gemm(ff, Lw["down_w"], packed_shape=(H, Lw["inter"]), out=o)
            K.rmsnorm(o, Lw["post_feedforward_layernorm"], eps, out=tmp)
            h.add_(tmp)
            if self.P:
                pg = self.ple_g[:T]
                K.gemm(h, Lw["ple_gate_w"], packed_shape=(self.P, H), act="gelu_tanh", out=pg)
                pg.mul_(self.ple[:T, g.idx * self.P:(g.idx + 1) * self.P])
                K.gemm(pg, Lw["ple_proj_w"], packed_shape=(H, self.P), out=o)
                K.rmsnorm(o, Lw["ple_norm"], eps, out=tmp)
                h.add_(tmp)
            if Lw["scalar"] != 1.0:
                h.mul_(Lw["scalar"])

    def _logits(self, rows_idx: torch.Tensor) -> torch.Tensor:
        K = self.K
        last = self.h.index_select(0, rows_idx.long())
        normed = K.rmsnorm(last, self.final_w, self.eps)
        logits = K.gemm(normed, self.lm_head).float()
        if self.softcap:
            logits = torch.tanh(logits / float(self.softcap)) * float(self.softcap)
        return logits

    # ------------------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def extend(self, tokens: Sequence[torch.Tensor], *, all_logits: bool = False) -> torch.Tensor:
        """Append ``tokens[b]`` to sequence ``b`` and return fp32 logits: ``[B, vocab]`` of the last rows, or with
        ``all_logits`` a list of ``[len_b, vocab]``."""
        B = len(tokens)
        lens = [int(t.numel()) for t in tokens]
        T = sum(lens)
        if B > self.B or T > self.T:
            raise RPUBackendError(f"{B} sequences / {T} rows exceed the engine's {self.B} / {self.T}")
        for b, n in enumerate(lens):
            if self.lengths[b] + n > self.S:
                raise RPUBackendError(f"sequence {b} would reach {self.lengths[b] + n} tokens, the cache holds {self.S}")
        dev = self.device
        ids = torch.cat([t.reshape(-1).to(torch.int32) for t in tokens]).to(dev)
        pos = torch.cat([torch.arange(self.lengths[b], self.lengths[b] + n, dtype=torch.int32) for b, n in enumerate(lens)])
        rows = torch.cat([pos[sum(lens[:b]):sum(lens[:b + 1])] + b * self.S for b in range(B)])
        starts = [sum(lens[:b]) for b in range(B)]
        meta = torch.tensor([starts, lens, [b * self.S for b in range(B)], [self.lengths[b] + lens[b] for b in range(B)]],
                            dtype=torch.int32).to(dev)
        self._run(T, ids, pos.to(dev), rows.to(dev), meta[0].contiguous(), meta[1].contiguous(), meta[2].contiguous(),
                  meta[3].contiguous(), max(lens))
        for b, n in enumerate(lens):
            self.lengths[b] += n
        if all_logits:
            full = self._logits(torch.arange(T, dtype=torch.int32, device=dev))
            return [full[starts[b]:starts[b] + lens[b]] for b in range(B)]
        return self._logits(torch.tensor([starts[b] + lens[b] - 1 for b in range(B)], dtype=torch.int32, device=dev))

    def prefill(self, tokens: Sequence[torch.Tensor], **kw):
        self.reset()
        return self.extend(tokens, **kw)

    # ---- greedy decode from a graph ----------------------------------------------------------------------------------
    def _decode_step(self, B: int) -> None:
        self._run(B, self.d_ids[:B], self.d_pos[:B], self.d_rows[:B], self.d_qstart[:B], self.d_qlen[:B], self.d_kvstart[:B],
                  self.d_kvlen[:B], 1)
        logits = self._logits(self.d_qstart[:B])
        nxt = logits.argmax(-1).to(torch.int32)
        self.d_next[:B].copy_(nxt)
        self.d_ids[:B].copy_(nxt)
        self.d_pos[:B].add_(1)
        self.d_rows[:B].add_(1)
        self.d_kvlen[:B].add_(1)

    @torch.no_grad()
    def decode(self, first: torch.Tensor, n_steps: int, *, use_graph: bool = True) -> torch.Tensor:
        """Feed ``first [B]`` (the token chosen after the last ``extend``) and generate ``n_steps`` greedy tokens: ``[B, n_steps]``."""
        B = int(first.numel())
        for b in range(B):
            if self.lengths[b] + n_steps > self.S:
                raise RPUBackendError(f"sequence {b} would outgrow the cache ({self.S})")
        dev = self.device
        lens = torch.tensor(self.lengths[:B], dtype=torch.int32)
        self.d_ids[:B].copy_(first.reshape(-1).to(dev, torch.int32))
        self.d_pos[:B].copy_(lens.to(dev))
        self.d_rows[:B].copy_((lens + torch.arange(B, dtype=torch.int32) * self.S).to(dev))
        self.d_kvlen[:B].copy_((lens + 1).to(dev))
        out = torch.empty((B, n_steps), dtype=torch.int32, device=dev)
        if use_graph and B not in self._graphs:
            snap = [t.clone() for t in (self.d_ids, self.d_pos, self.d_rows, self.d_kvlen)]
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                self._decode_step(B)
            torch.cuda.current_stream().wait_stream(st)
            for dst, src in zip((self.d_ids, self.d_pos, self.d_rows, self.d_kvlen), snap):
                dst.copy_(src)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                self._decode_step(B)
            torch.cuda.synchronize()
            for dst, src in zip((self.d_ids, self.d_pos, self.d_rows, self.d_kvlen), snap):
                dst.copy_(src)
            self._graphs[B] = g
        for i in range(n_steps):
            if use_graph:
                self._graphs[B].replay()
            else:
                self._decode_step(B)
            out[:, i].copy_(self.d_next[:B])
        for b in range(B):
            self.lengths[b] += n_steps
        return out

    @torch.no_grad()
    def generate(self, tokens: Sequence[torch.Tensor], max_new_tokens: int) -> torch.Tensor:
        logits = self.prefill(tokens)
        first = logits.argmax(-1).to(torch.int32)
        if max_new_tokens <= 1:
            return first[:, None]
        rest = self.decode(first, max_new_tokens - 1)
        self.check_status()
        return torch.cat((first[:, None], rest), 1)

    def check_status(self) -> None:
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")

    def close(self) -> None:
        self._graphs.clear()


__all__ = ["Gemma4Engine", "rope_tables", "preflight"]
