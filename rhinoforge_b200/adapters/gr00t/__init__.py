"""GR00T-N1.7 adapter: checkpoint directory -> :class:`Gr00tN1d7VLA` (image + text + state -> a 40 x 132 action chunk).

The checkpoint is a standalone bundle, not a ``transformers`` model: ``backbone.model.*`` holds a Qwen3-VL whose language
model is cut after layer 16, ``action_head.*`` the VL encoder, the DiT and the per-embodiment encoder / decoder banks.
``build_gr00t_vla`` therefore has its own builder: the backbone becomes a :class:`Qwen3VLEngine` with a 16-layer text
config (its residual stream after the last layer - before the final RMSNorm - is what the action head reads), the head a
:class:`rhinoforge_b200.models.gr00t.Gr00tEngine`.

``get_action(inputs, seed=, num_steps=)`` takes the processor's ``input_ids``, ``attention_mask``, ``pixel_values``,
``image_grid_thw`` and ``state`` and returns the normalised action chunk ``[1, 40, 132]`` fp32 on the host; the initial
noise is drawn on the host from ``seed``.

Reference: ``python/rpu_backend/adapters/gr00t/runtime.py:466-530,1016-1048`` (runtime object and ``get_action``),
``:1230-1250,1330-1370`` (builder: truncated backbone, key prefix, missing-weight guard).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Callable, Dict, Mapping, Optional

import torch

from ...api.errors import UnsupportedModelError
from ...models.gr00t import AP, Gr00tConfig, Gr00tEngine

SELECT_LAYER = 16
BACKBONE_PREFIX = "backbone.model."


def checkpoint_reader(ckpt_path: str) -> Callable[[str], torch.Tensor]:
    """``get(name)`` over a sharded safetensors directory (``*.index.json`` weight map) or a single file."""
    from safetensors import safe_open
    index = glob.glob(os.path.join(ckpt_path, "*.index.json"))
    if index:
        with open(index[0]) as f:
            wmap = json.load(f)["weight_map"]
    else:
        wmap = {}
        for path in sorted(glob.glob(os.path.join(ckpt_path, "*.safetensors"))):
            with safe_open(path, framework="pt") as sf:
                for k in sf.keys():
                    wmap[k] = os.path.basename(path)
    if not wmap:
        raise ValueError(f"no safetensors weights under {ckpt_path}")
    handles: Dict[str, object] = {}

    def get(name: str) -> torch.Tensor:
        shard = wmap[name]                     # KeyError names the missing tensor
        if shard not in handles:
            handles[shard] = safe_open(os.path.join(ckpt_path, shard), framework="pt")
        return handles[shard].get_tensor(name)
    get.names = set(wmap)
    return get


def head_config_from(action_head_cfg: Optional[Mapping], get, **overrides) -> Gr00tConfig:
    """Geometry from the bundle's ``action_head_cfg`` where present, else from the tensors themselves."""
    c = dict(action_head_cfg or {})
    kw = {}
    w1 = get(AP + "action_encoder.W1.W")
    kw.update(embodiments=w1.shape[0], action_dim=w1.shape[1], hidden=w1.shape[2])
    kw["state_dim"], kw["enc_mid"] = get(AP + "state_encoder.layer1.W").shape[1:]
    kw["model_out"], kw["dec_mid"] = get(AP + "action_decoder.layer1.W").shape[1:]
    kw["max_pos"] = get(AP + "position_embedding.weight").shape[0]
    kw["vl_dim"] = get(AP + "vlln.weight").shape[0]
    kw["ff"] = get(AP + "model.transformer_blocks.0.ff.net.0.proj.weight").shape[0]
    kw["vl_ff"] = get(AP + "vl_self_attention.transformer_blocks.0.ff.net.0.proj.weight").shape[0]
    kw["time_embed"] = get(AP + "model.timestep_encoder.timestep_embedder.linear_1.weight").shape[1]
    names = getattr(get, "names", None)
    if names is not None:
        count = lambda p: len({n[len(p):].split(".")[0] for n in names if n.startswith(p)})
        kw["layers"] = count(AP + "model.transformer_blocks.")
        kw["vl_layers"] = count(AP + "vl_self_attention.transformer_blocks.")
    dit = c.get("diffusion_model_cfg", {})
    if "num_attention_heads" in dit:
        kw["heads"], kw["head_dim"] = dit["num_attention_heads"], dit.get("attention_head_dim", kw["hidden"] // dit["num_attention_heads"])
    vl = c.get("vl_self_attention_cfg", {})
    if "num_attention_heads" in vl:
        kw["vl_heads"], kw["vl_head_dim"] = vl["num_attention_heads"], vl.get("attention_head_dim", kw["vl_dim"] // vl["num_attention_heads"])
    for src, dst in (("action_horizon", "horizon"), ("num_inference_timesteps", "steps"), ("num_timestep_buckets", "buckets")):
        if src in c:
            kw[dst] = c[src]
    kw.update(overrides)
    cfg = Gr00tConfig(**kw)
    if cfg.heads * cfg.head_dim != cfg.hidden or cfg.vl_heads * cfg.vl_head_dim != cfg.vl_dim:
        raise UnsupportedModelError(f"GR00T head geometry {cfg.heads} x {cfg.head_dim} / {cfg.vl_heads} x {cfg.vl_head_dim} does not "
                                    f"tile the widths {cfg.hidden} / {cfg.vl_dim}")
    return cfg


class Gr00tN1d7VLA:
    def __init__(self, backbone, head: Gr00tEngine, *, image_token_id: int, embodiment_id: int):
        self.backbone, self.head, self.image_token_id, self.embodiment_id = backbone, head, image_token_id, embodiment_id
        self.cfg = head.cfg

    @torch.no_grad()
    def backbone_hidden(self, inputs: Mapping) -> torch.Tensor:
        """Residual stream ``[S, vl_dim]`` after the backbone's last (16th) layer, on the device."""
        ids = inputs["input_ids"].reshape(-1)
        self.backbone.prefill(ids, inputs.get("pixel_values"), inputs.get("image_grid_thw"))
        return self.backbone.text.hidden[:ids.numel()]

    @torch.no_grad()
    def get_action(self, inputs: Mapping, *, seed: int = 0, num_steps: Optional[int] = None) -> torch.Tensor:
        cfg = self.cfg
        if num_steps is not None and num_steps != cfg.steps:
            raise ValueError(f"the denoise tables are built for num_steps={cfg.steps}; got {num_steps}. Rebuild for another schedule.")
        ids = inputs["input_ids"].reshape(-1)
        S = int(ids.numel())
        cap = min(self.head.max_vl, self.backbone.text.max_tokens, self.backbone.text.cache.max_seq_len - 1)
        if S > cap:
            raise ValueError(f"GR00T input of {S} tokens exceeds the built capacity {cap}; rebuild with a larger max_vl")
        valid = inputs.get("attention_mask")
        valid = torch.ones(S, dtype=torch.bool) if valid is None else (valid.reshape(-1) == 1)
        if not bool(valid.all()):
            raise ValueError("padded prompts are not supported: pass one unpadded sequence")
        hidden = self.backbone_hidden(inputs)
        vl = self.head.vl_encode(hidden)
        noise = torch.randn(1, cfg.horizon, cfg.action_dim, generator=torch.Generator().manual_seed(int(seed)))
        state = inputs["state"].reshape(-1).float()
        if state.numel() > cfg.state_dim:
            raise ValueError(f"state has {state.numel()} values, the encoder takes {cfg.state_dim}")
        state = torch.nn.functional.pad(state, (0, cfg.state_dim - state.numel()))
        act = self.head.denoise(vl, state, noise[0], ids.cpu() == self.image_token_id, valid)
        self.head.check_status()
        self.backbone.text.check_status()
        return act.cpu().reshape(1, cfg.horizon, cfg.action_dim)

    def close(self) -> None:
        self.head.close()
        self.backbone.close()


def backbone_getter(get, *, prefix: str = BACKBONE_PREFIX):
    """Hugging Face Qwen3-VL names over the bundle's ``backbone.model.*`` tensors; the cut language model has no output
    head of its own, so ``lm_head.weight`` resolves to the token embedding."""
    names = getattr(get, "names", None)

    def g(name: str) -> torch.Tensor:
        if name == "lm_head.weight":
            name = "model.language_model.embed_tokens.weight"
        return get(prefix + name)
    if names is not None:
        g.names = {n[len(prefix):] for n in names if n.startswith(prefix)} | {"lm_head.weight"}
        if not any(n.startswith("model.language_model.layers.") for n in g.names):
            raise ValueError(f"no `{prefix}*` language-model tensors in the bundle (wrong bundle or changed prefix)")
    return g


def build_gr00t_vla(ckpt_path: str, qwen3vl_local: str, *, embodiment_id: int = 20, max_vl: int = 512, device="cuda",
                    dtype=torch.float16, num_steps: Optional[int] = None, select_layer: int = SELECT_LAYER,
                    max_patches: int = 4096, head_overrides: Optional[Mapping] = None) -> Gr00tN1d7VLA:
    """``ckpt_path``: the GR00T bundle; ``qwen3vl_local``: a directory with the Qwen3-VL ``config.json`` the backbone was
    derived from; ``select_layer``: the language-model layer whose output the action head reads (the layers after it
    are not loaded)."""
    from transformers import Qwen3VLConfig
    from ...models.qwen3_vl import Qwen3VLEngine
    get = checkpoint_reader(ckpt_path)
    hf = Qwen3VLConfig.from_pretrained(qwen3vl_local)
    hf.text_config.num_hidden_layers = select_layer
    bundle_cfg = {}
    cfg_path = os.path.join(ckpt_path, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            bundle_cfg = json.load(f).get("action_head_cfg", {})
    overrides = dict(head_overrides or {})
    if num_steps is not None:
        overrides["steps"] = num_steps
    cfg = head_config_from(bundle_cfg, get, **overrides)
    if cfg.vl_dim != hf.text_config.hidden_size:
        raise UnsupportedModelError(f"the action head reads {cfg.vl_dim}-wide tokens, the backbone emits {hf.text_config.hidden_size}")
    bget = backbone_getter(get)
    missing = [f"model.language_model.layers.{i}.self_attn.q_proj.weight" for i in range(select_layer)
               if f"model.language_model.layers.{i}.self_attn.q_proj.weight" not in bget.names]
    if missing:
        raise ValueError(f"GR00T backbone: {len(missing)} of {select_layer} layers have no weights in the bundle (e.g. {missing[:2]})")
    backbone = Qwen3VLEngine(hf, bget, device=device, dtype=dtype, max_seq_len=max_vl + 16, max_batch=1, max_prefill_tokens=max_vl,
                             max_patches=max_patches, names=bget.names)
    try:
        head = Gr00tEngine(cfg, get, embodiment=embodiment_id, max_vl=max_vl, device=device, dtype=dtype)
    except BaseException:
        backbone.close()
        raise
    return Gr00tN1d7VLA(backbone, head, image_token_id=hf.image_token_id, embodiment_id=embodiment_id)


__all__ = ["Gr00tN1d7VLA", "build_gr00t_vla", "checkpoint_reader", "head_config_from", "backbone_getter", "SELECT_LAYER"]
