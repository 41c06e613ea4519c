"""W8A16 / W4 quantisation helpers, the offline converter and the loader layout (CPU)."""
import json
from pathlib import Path

import pytest
import torch


def test_per_channel_int8_quantisation():
    from rpu_backend.quant._common import (cosine, dequantize_linear_per_channel, quantize_linear_per_channel,
                                           reference_linear)
    w = torch.randn(64, 128) * 0.05
    q, s = quantize_linear_per_channel(w)
    assert q.dtype == torch.int8 and int(q.min()) >= -127 and int(q.max()) <= 127
    assert s.dtype == torch.float16 and s.shape == (64,)
    assert cosine(dequantize_linear_per_channel(q, s), w) > 0.999
    x = torch.randn(5, 128)
    assert cosine(reference_linear(x, q, s), x @ w.t()) > 0.999
    with pytest.raises(ValueError):
        quantize_linear_per_channel(torch.randn(3))


def test_w8a16_config_marker():
    from types import SimpleNamespace
    from rpu_backend.quant.load import is_w8a16_config
    assert is_w8a16_config(SimpleNamespace(quant_config={"method": "w8a16"}))
    assert not is_w8a16_config(SimpleNamespace(quant_config={"method": "gptq"}))
    assert not is_w8a16_config(SimpleNamespace())


def test_int4_and_nvfp4_packers_round_trip():
    from rpu_backend.quant.int4_pack import pack_int4, quantize_pack_int4, unpack_int4
    from rpu_backend.quant.int4_pgrp_pack import dequantize_int4_pgrp, quantize_pack_int4_pgrp
    from rpu_backend.quant.nvfp4_pack import dequantize_nvfp4, quantize_nvfp4
    from rpu_backend.quant._common import cosine
    q = torch.randint(-8, 8, (7, 64), dtype=torch.int8)
    assert torch.equal(unpack_int4(pack_int4(q)), q)
    w = torch.randn(32, 128) * 0.1
    p, s = quantize_pack_int4(w)
    assert p.shape == (32, 64) and s.shape == (32,)
    pg, sg = quantize_pack_int4_pgrp(w, 32)
    assert sg.shape == (32, 4) and cosine(dequantize_int4_pgrp(pg, sg, 32), w) > 0.98
    codes, bs, ts = quantize_nvfp4(w)
    assert codes.shape == (32, 128) and bs.shape == (8, 32) and bs.dtype == torch.uint8     # scales are [K/16, N]
    deq = dequantize_nvfp4(codes, bs, ts)
    assert deq.dtype == torch.float32 and cosine(deq, w) > 0.97


def test_nvfp4_encoder_rounds_ties_to_the_even_code_and_keeps_signed_zero():
    from rpu_backend.quant.nvfp4_pack import (fp4_e2m1_decode, fp4_e2m1_encode, pack_nibbles, quantize_nvfp4,
                                              unpack_nibbles)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert fp4_e2m1_decode(fp4_e2m1_encode(ties)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    assert fp4_e2m1_decode(fp4_e2m1_encode(-ties)).tolist() == [-0.0, -1.0, -1.0, -2.0, -2.0, -4.0, -4.0]
    off = torch.tensor([0.26, 0.74, 1.26, 1.74, 2.51, 3.49, 5.01, 100.0])
    assert fp4_e2m1_decode(fp4_e2m1_encode(off)).tolist() == [0.5, 0.5, 1.5, 1.5, 3.0, 3.0, 6.0, 6.0]
    assert int(fp4_e2m1_encode(torch.tensor([-0.0]))[0]) == 8                      # sign bit survives on -0.0
    zero = torch.zeros(2, 32)
    codes, scales, ts = quantize_nvfp4(zero)
    assert float(ts) == 2.0 ** -24 and int(codes.max()) == 0 and int(scales.max()) == 0
    c = torch.randint(0, 16, (3, 32), dtype=torch.uint8)
    assert torch.equal(unpack_nibbles(pack_nibbles(c)), c)


def _tiny_ckpt(path: Path, tie=True):
    from safetensors.torch import save_file
    from transformers import Qwen3Config
    from rhinoforge_b200.models.decoder import random_state_dict, tiny_config
    cfg = tiny_config(tie_embeddings=tie)
    hf = Qwen3Config(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                     num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_heads,
                     num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, tie_word_embeddings=tie,
                     max_position_embeddings=512, architectures=["Qwen3ForCausalLM"])
    path.mkdir(parents=True)
    hf.save_pretrained(path)
    sd = random_state_dict(cfg, dtype=torch.float16)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(path / "model.safetensors"), metadata={"format": "pt"})
    (path / "tokenizer_config.json").write_text("{}")
    return cfg, sd


def test_converter_layout_and_refusal_to_overwrite(tmp_path):
    from safetensors.torch import load_file
    from rpu_backend.quant.convert_qwen3 import convert_checkpoint, main
    from rpu_backend.quant._common import cosine, dequantize_linear_per_channel
    cfg, sd = _tiny_ckpt(tmp_path / "src", tie=True)
    stats = convert_checkpoint(tmp_path / "src", tmp_path / "dst", ["lm_head"], quant_lm_head=True)
    assert stats["n_quantized"] == 7 * cfg.num_layers + 1
    out = load_file(str(tmp_path / "dst" / "model.safetensors"))
    name = "model.layers.0.mlp.down_proj.weight"
    assert out[name].dtype == torch.int8 and out["model.layers.0.mlp.down_proj.weight_scale"].dtype == torch.float16
    assert cosine(dequantize_linear_per_channel(out[name], out[name[:-7] + ".weight_scale"]), sd[name]) > 0.999
    assert out["lm_head.weight"].dtype == torch.int8 and out["model.embed_tokens.weight"].dtype == torch.float16
    assert out["model.layers.0.input_layernorm.weight"].dtype == torch.float16
    qc = json.loads((tmp_path / "dst" / "config.json").read_text())["quant_config"]
    assert qc == {"method": "w8a16", "mode": "per_channel_symmetric", "qaxis": 0, "skip_modules": [],
                  "quantized_lm_head": True, "quantized_embed_tokens": False, "lm_head_untied": True,
                  "embed_tokens_untied": False}
    assert (tmp_path / "dst" / "tokenizer_config.json").is_file()
    assert main(["--src", str(tmp_path / "src"), "--dst", str(tmp_path / "dst")]) == 1
    assert main(["--src", str(tmp_path / "src"), "--dst", str(tmp_path / "d2"), "--quant-embed-tokens"]) == 1
    assert not list(tmp_path.glob(".*tmp*"))


def test_w8a16_loader_keeps_int8_parameters(tmp_path):
    from transformers import AutoConfig
    from rpu_backend.quant.convert_qwen3 import convert_checkpoint
    from rpu_backend.quant.load import is_w8a16_config, load_w8a16_model, w8a16_tensor_getter
    _tiny_ckpt(tmp_path / "src", tie=False)
    convert_checkpoint(tmp_path / "src", tmp_path / "dst", ["lm_head"])
    config = AutoConfig.from_pretrained(tmp_path / "dst")
    assert is_w8a16_config(config)
    model = load_w8a16_model(config, str(tmp_path / "dst"))
    lin = model.model.layers[0].self_attn.q_proj
    assert lin.weight.dtype == torch.int8 and lin.weight_scale.dtype == torch.float16
    assert model.lm_head.weight.dtype == torch.float16
    get = w8a16_tensor_getter(str(tmp_path / "dst"))
    assert get("model.layers.1.mlp.up_proj.weight").dtype == torch.int8
    assert get.scale("model.layers.1.mlp.up_proj.weight").shape == (512,)
    assert get.scale("model.norm.weight") is None


def test_w8a16_loader_refuses_mis_sized_half_converted_and_mis_scaled_checkpoints(tmp_path):
    from safetensors.torch import load_file, save_file
    from transformers import AutoConfig
    from rpu_backend.quant.convert_qwen3 import convert_checkpoint
    from rpu_backend.quant.load import load_w8a16_model
    _tiny_ckpt(tmp_path / "src", tie=False)
    convert_checkpoint(tmp_path / "src", tmp_path / "dst", ["lm_head"])
    config = AutoConfig.from_pretrained(tmp_path / "dst")
    good = load_file(str(tmp_path / "dst" / "model.safetensors"))
    qname = "model.layers.0.self_attn.q_proj.weight"

    def variant(tag, edit):
        d = tmp_path / tag
        d.mkdir()
        (d / "config.json").write_text((tmp_path / "dst" / "config.json").read_text())
        t = {k: v.clone() for k, v in good.items()}
        edit(t)
        save_file(t, str(d / "model.safetensors"), metadata={"format": "pt"})
        return str(d)

    with pytest.raises(ValueError, match="the model expects"):                     # a row short
        load_w8a16_model(config, variant("short", lambda t: t.__setitem__(qname, t[qname][:-1].contiguous())))
    with pytest.raises(TypeError, match="must be int8"):                           # projection left in 16 bits
        load_w8a16_model(config, variant("half", lambda t: t.__setitem__(qname, t[qname].to(torch.float16))))
    with pytest.raises(ValueError, match="one entry per output row"):              # scale of the wrong length
        load_w8a16_model(config, variant("scale", lambda t: t.__setitem__(qname + "_scale", t[qname + "_scale"][:-1].contiguous())))
    with pytest.raises(ValueError, match="must be fp16"):                          # scale of the wrong dtype
        load_w8a16_model(config, variant("sdtype", lambda t: t.__setitem__(qname + "_scale", t[qname + "_scale"].float())))


def test_verify_accepts_a_converted_checkpoint_and_flags_a_corrupted_one(tmp_path):
    from safetensors.torch import load_file, save_file
    from rpu_backend.quant.convert_qwen3 import convert_checkpoint
    from rpu_backend.quant.verify_qwen3_w8a16 import main, verify
    _tiny_ckpt(tmp_path / "src", tie=False)
    convert_checkpoint(tmp_path / "src", tmp_path / "q", ["lm_head"])
    rep = verify(tmp_path / "src", tmp_path / "q")
    assert rep["ok"] and rep["quantized"] > 0 and rep["worst_cosine"] > 0.999 and rep["worst_rel_product_error"] < 0.02
    assert main(["--src", str(tmp_path / "src"), "--quant", str(tmp_path / "q")]) == 0
    t = load_file(str(tmp_path / "q" / "model.safetensors"))
    name = "model.layers.0.self_attn.q_proj.weight"
    t[name] = t[name].clone()
    t[name][0, :8] = 127                                     # corrupt one row
    save_file(t, str(tmp_path / "q" / "model.safetensors"), metadata={"format": "pt"})
    rep = verify(tmp_path / "src", tmp_path / "q")
    assert not rep["ok"] and any(name in p for p in rep["problems"])
    assert main(["--src", str(tmp_path / "src"), "--quant", str(tmp_path / "q")]) == 1


def test_w4a16_converter_packs_projections_with_group_scales(tmp_path):
    from safetensors.torch import load_file
    from rpu_backend.quant.convert_qwen3_w4a16 import convert_checkpoint, main
    from rpu_backend.quant.int4_pgrp_pack import dequantize_int4_pgrp
    from rpu_backend.quant._common import cosine
    cfg, sd = _tiny_ckpt(tmp_path / "src", tie=False)
    st = convert_checkpoint(tmp_path / "src", tmp_path / "w4", group_size=32)
    assert st["n_quantized"] == 7 * cfg.num_layers
    out = load_file(str(tmp_path / "w4" / "model.safetensors"))
    name = "model.layers.1.mlp.up_proj.weight"
    w = sd[name]
    assert out[name].dtype == torch.uint8 and tuple(out[name].shape) == (w.shape[0], w.shape[1] // 2)
    sc = out[name[:-7] + ".weight_scale"]
    assert sc.dtype == torch.float16 and tuple(sc.shape) == (w.shape[0], w.shape[1] // 32)
    assert cosine(dequantize_int4_pgrp(out[name], sc, 32), w) > 0.99
    qc = json.loads((tmp_path / "w4" / "config.json").read_text())["quant_config"]
    assert qc["method"] == "w4a16" and qc["group_size"] == 32
    assert main(["--src", str(tmp_path / "src"), "--dst", str(tmp_path / "w4")]) == 1      # never overwrites


def test_pi05_converter_quantises_only_gemma_projections_and_writes_the_sidecar(tmp_path):
    from safetensors.torch import load_file, save_file
    from rpu_backend.quant.convert_pi05 import SIDECAR, convert_checkpoint, target_of
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    vlm = "model.paligemma_with_expert.paligemma.model.language_model.layers.0."
    exp = "model.paligemma_with_expert.gemma_expert.model.layers.0."
    sd = {vlm + "self_attn.q_proj.weight": r(32, 16), vlm + "mlp.down_proj.weight": r(16, 64),
          exp + "self_attn.o_proj.weight": r(16, 32), exp + "input_layernorm.dense.weight": r(48, 16),
          "model.paligemma_with_expert.paligemma.model.vision_tower.vision_model.encoder.layers.0.self_attn.q_proj.weight": r(16, 16),
          "model.action_in_proj.weight": r(16, 8)}
    src = tmp_path / "src"
    src.mkdir()
    save_file(sd, str(src / "model.safetensors"), metadata={"format": "pt"})
    (src / "config.json").write_text(json.dumps({"type": "pi05"}))
    (src / "model_remapped.safetensors").write_bytes(b"stale")
    assert target_of(vlm + "self_attn.q_proj.weight") == "vlm" and target_of(exp + "self_attn.o_proj.weight") == "expert"
    assert target_of(exp + "input_layernorm.dense.weight") is None
    st = convert_checkpoint(src, tmp_path / "q8")
    assert (st["vlm"], st["expert"], st["int8"]) == (2, 1, 3)
    out = load_file(str(tmp_path / "q8" / "model.safetensors"))
    assert out[vlm + "self_attn.q_proj.weight"].dtype == torch.int8
    assert out[vlm + "self_attn.q_proj.weight_scale"].dtype == torch.float16
    assert out[exp + "input_layernorm.dense.weight"].dtype == torch.float32          # untouched
    assert out["model.action_in_proj.weight"].dtype == torch.float32
    assert not (tmp_path / "q8" / "model_remapped.safetensors").exists()
    side = json.loads((tmp_path / "q8" / SIDECAR).read_text())
    assert side["method"] == "w8a16" and side["targets"] == ["vlm", "expert"]
    st4 = convert_checkpoint(src, tmp_path / "q4", bits=4, targets=["expert"], keep_int8_suffixes=["self_attn.o_proj"])
    out4 = load_file(str(tmp_path / "q4" / "model.safetensors"))
    assert (st4["expert"], st4["vlm"], st4["int8"], st4["int4"]) == (1, 0, 1, 0)     # the only expert tensor is exempt
    assert out4[vlm + "self_attn.q_proj.weight"].dtype == torch.float32
    st4b = convert_checkpoint(src, tmp_path / "q4b", bits=4)
    q = load_file(str(tmp_path / "q4b" / "model.safetensors"))[vlm + "mlp.down_proj.weight"]
    assert st4b["int4"] == 3 and int(q.max()) <= 7 and int(q.min()) >= -8


def test_wall_oss_converters_scope_and_sidecars(tmp_path):
    """W8A16: every 2-D weight but the token embedding.  W4A16: only the fused expert projections of the decoder, as
    4-bit values in int8 containers or packed groups; `--keep-int8` retreats a suffix to 8 bits."""
    from safetensors.torch import load_file, save_file
    from rpu_backend.quant.convert_wall_oss import convert_checkpoint as to_w4
    from rpu_backend.quant.convert_wall_oss_w8a16 import convert_checkpoint as to_w8, main as main_w8
    from rpu_backend.quant.int4_pgrp_pack import dequantize_int4_pgrp
    from rpu_backend.quant._common import cosine, dequantize_linear_per_channel
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    L = "model.layers.0."
    sd = {"model.embed_tokens.weight": r(40, 32), L + "self_attn.qkv_proj_experts.0.weight": r(96, 32),
          L + "self_attn.o_proj_experts.1.weight": r(32, 32), L + "moe.experts.0.gate_up_proj.weight": r(128, 32),
          L + "moe.experts.1.down_proj.weight": r(32, 64), L + "input_layernorm.weight": r(32),
          "visual.blocks.0.attn.qkv.weight": r(96, 32), "visual.blocks.0.attn.qkv.bias": r(96),
          "action_preprocessor.proj.weight": r(32, 16)}
    src = tmp_path / "src"
    src.mkdir()
    save_file(sd, str(src / "model.safetensors"), metadata={"format": "pt"})
    (src / "config.json").write_text("{}")
    (src / "norm_stats.json").write_text("{}")
    st = to_w8(src, tmp_path / "w8")
    out = load_file(str(tmp_path / "w8" / "model.safetensors"))
    assert st["n_quantized"] == 6                                        # all 2-D weights except the embedding
    assert out["model.embed_tokens.weight"].dtype == torch.float32 and out["visual.blocks.0.attn.qkv.weight"].dtype == torch.int8
    assert out["visual.blocks.0.attn.qkv.bias"].dtype == torch.float32
    name = "action_preprocessor.proj.weight"
    assert cosine(dequantize_linear_per_channel(out[name], out[name[:-7] + ".weight_scale"]), sd[name]) > 0.999
    side = json.loads((tmp_path / "w8" / "rpu_quant_config.json").read_text())
    assert side["method"] == "w8a16" and side["skip_modules"] == ["embed_tokens"]
    assert (tmp_path / "w8" / "norm_stats.json").is_file()
    assert main_w8(["--src", str(src), "--dst", str(tmp_path / "w8")]) == 1                  # never overwrites
    st4 = to_w4(src, tmp_path / "w4", keep_int8=["self_attn.o_proj_experts.1"])
    o4 = load_file(str(tmp_path / "w4" / "model.safetensors"))
    assert (st4["int4"], st4["int8"]) == (3, 1)
    q = o4[L + "moe.experts.0.gate_up_proj.weight"]
    assert q.dtype == torch.int8 and int(q.max()) <= 7 and int(q.min()) >= -8
    assert int(o4[L + "self_attn.o_proj_experts.1.weight"].abs().max()) > 8            # kept at 8 bits
    assert o4["visual.blocks.0.attn.qkv.weight"].dtype == torch.float32                  # vision untouched
    stg = to_w4(src, tmp_path / "w4g", group_size=32)
    og = load_file(str(tmp_path / "w4g" / "model.safetensors"))
    name = L + "moe.experts.1.down_proj.weight"
    assert og[name].dtype == torch.uint8 and tuple(og[name].shape) == (32, 32) and stg["int4"] == 4
    assert cosine(dequantize_int4_pgrp(og[name], og[name[:-7] + ".weight_scale"], 32), sd[name]) > 0.99
    assert json.loads((tmp_path / "w4g" / "rpu_quant_config.json").read_text())["group_size"] == 32


def test_w4a16_checkpoint_is_dequantised_when_read(tmp_path):
    from rpu_backend.quant._common import cosine
    from rpu_backend.quant.convert_qwen3_w4a16 import convert_checkpoint
    from rpu_backend.quant.load import is_w4a16_config, w4a16_tensor_getter
    cfg, sd = _tiny_ckpt(tmp_path / "src", tie=False)
    convert_checkpoint(tmp_path / "src", tmp_path / "w4", group_size=32)
    config = json.loads((tmp_path / "w4" / "config.json").read_text())
    assert is_w4a16_config(config) and not is_w4a16_config({"quant_config": {"method": "w8a16"}})
    get = w4a16_tensor_getter(str(tmp_path / "w4"), config)
    name = "model.layers.0.self_attn.q_proj.weight"
    w = get(name)
    assert w.dtype == torch.float16 and w.shape == sd[name].shape and cosine(w, sd[name]) > 0.99
    assert get("model.layers.0.input_layernorm.weight").dtype == torch.float16
    assert not any(n.endswith(".weight_scale") for n in get.names) and name in get.names


def test_wall_oss_checkpoint_pair_validation(tmp_path):
    """A converted directory is accepted only with the 16-bit directory it was converted from."""
    from safetensors.torch import save_file
    from rpu_backend.quant.checkpoint_pair import (validate_checkpoint_pair, validate_rtc_w4_checkpoint_pair,
                                                   validate_w8_nvfp4_checkpoint_pair)
    from rpu_backend.quant.convert_wall_oss import QUANT_SUFFIXES, convert_checkpoint as to_w4
    from rpu_backend.quant.convert_wall_oss_w8a16 import convert_checkpoint as to_w8
    g = torch.Generator().manual_seed(1)
    L = "model.layers.0."
    sd = {L + s: torch.randn(64, 64, generator=g) * 0.05 for s in QUANT_SUFFIXES}
    sd["model.embed_tokens.weight"] = torch.randn(16, 64, generator=g)

    def make_src(path, **cfg):
        path.mkdir()
        save_file(sd, str(path / "model.safetensors"), metadata={"format": "pt"})
        (path / "config.json").write_text(json.dumps({"hidden_size": 64, "num_hidden_layers": 1, "torch_dtype": "bfloat16",
                                                      **cfg}))
        return path

    src = make_src(tmp_path / "wall-oss")
    other = make_src(tmp_path / "wall-oss-finetune")
    bigger = make_src(tmp_path / "wall-oss-big", hidden_size=128)
    to_w8(src, tmp_path / "w8")
    cfg = json.loads((tmp_path / "w8" / "config.json").read_text())
    cfg["torch_dtype"] = "float16"                                     # a representation field may differ
    (tmp_path / "w8" / "config.json").write_text(json.dumps(cfg))
    qcfg, fcfg = validate_w8_nvfp4_checkpoint_pair(tmp_path / "w8", src)
    assert qcfg["hidden_size"] == fcfg["hidden_size"] == 64
    assert json.loads((tmp_path / "w8" / "rpu_quant_config.json").read_text())["source"] == "wall-oss"   # name, not a path

    with pytest.raises(ValueError, match="not a declared source pair"):
        validate_w8_nvfp4_checkpoint_pair(tmp_path / "w8", other)
    with pytest.raises(ValueError, match="got unquantized"):
        validate_w8_nvfp4_checkpoint_pair(src, src)                     # arguments of the wrong kind
    with pytest.raises(ValueError, match="must be an unquantized source"):
        validate_w8_nvfp4_checkpoint_pair(tmp_path / "w8", tmp_path / "w8")
    with pytest.raises(ValueError, match="method='w4a16'; got w8a16"):
        validate_rtc_w4_checkpoint_pair(tmp_path / "w8", src)

    # a converted directory that was moved away from its source cannot be resolved
    moved = tmp_path / "elsewhere"
    moved.mkdir()
    (tmp_path / "w8").rename(moved / "w8")
    with pytest.raises(ValueError, match="cannot be resolved exactly"):
        validate_w8_nvfp4_checkpoint_pair(moved / "w8", src)
    side = json.loads((moved / "w8" / "rpu_quant_config.json").read_text())
    (moved / "w8" / "rpu_quant_config.json").write_text(json.dumps({**side, "source": str(src)}))  # absolute is allowed
    validate_w8_nvfp4_checkpoint_pair(moved / "w8", src)
    (moved / "w8" / "rpu_quant_config.json").write_text(json.dumps({k: v for k, v in side.items() if k != "source"}))
    with pytest.raises(ValueError, match="no source provenance"):
        validate_w8_nvfp4_checkpoint_pair(moved / "w8", src)

    # same provenance, different architecture fields
    to_w8(bigger, tmp_path / "w8big")
    cfgb = json.loads((tmp_path / "w8big" / "config.json").read_text())
    (tmp_path / "w8big" / "config.json").write_text(json.dumps({**cfgb, "hidden_size": 64, "rope_theta": 5.0}))
    with pytest.raises(ValueError, match=r"mismatched config fields: \['hidden_size', 'rope_theta'\]"):
        validate_w8_nvfp4_checkpoint_pair(tmp_path / "w8big", bigger)

    # sidecar and embedded record must agree
    (tmp_path / "w8big" / "config.json").write_text(json.dumps({**cfgb, "quant_config": {"method": "w4a16"}}))
    with pytest.raises(ValueError, match="conflicting quantization metadata"):
        validate_w8_nvfp4_checkpoint_pair(tmp_path / "w8big", bigger)

    # the real-time-chunking composition: group 32, expert-0 down projection kept at 8 bits, nothing else
    to_w4(src, tmp_path / "rtc", keep_int8=["moe.experts.0.down_proj"], group_size=32)
    validate_rtc_w4_checkpoint_pair(tmp_path / "rtc", src)
    to_w4(src, tmp_path / "w4_plain", group_size=32)
    with pytest.raises(ValueError, match="exact seven group-wise INT4"):
        validate_rtc_w4_checkpoint_pair(tmp_path / "w4_plain", src)
    to_w4(src, tmp_path / "w4_g64", keep_int8=["moe.experts.0.down_proj"], group_size=64)
    with pytest.raises(ValueError, match="group_size=32"):
        validate_rtc_w4_checkpoint_pair(tmp_path / "w4_g64", src)
    assert validate_checkpoint_pair(tmp_path / "w4_plain", src, expected_method="w4a16", label="W4A16")[2]["group_size"] == 32


def test_w8a16_inventory_is_checked_from_headers_alone(tmp_path):
    """The real converter's output passes; each way of being almost right is named."""
    from safetensors.torch import load_file, save_file
    from rpu_backend.quant.convert_qwen3 import convert_checkpoint
    from rpu_backend.quant.inventory import inspect_w8a16_checkpoint, is_decoder_projection
    cfg, sd = _tiny_ckpt(tmp_path / "src", tie=False)
    convert_checkpoint(tmp_path / "src", tmp_path / "w8", ["lm_head"])
    plan = inspect_w8a16_checkpoint(tmp_path / "w8")
    assert len(plan["int8"]) == len(plan["scales"]) == 7 * cfg.num_layers and not plan["unquantized"]
    assert len(plan["layers"]) == cfg.num_layers and "model.embed_tokens.weight" in plan["nondecoder"]
    assert all(any(n.endswith("q_proj.weight_scale") for n in names) for names in plan["layers"])
    assert set(plan["tensor_shards"].values()) == {"model.safetensors"} and plan["bytes"] > 0
    assert is_decoder_projection("model.language_model.layers.3.mlp.up_proj.weight")
    assert not is_decoder_projection("model.visual.blocks.3.mlp.up_proj.weight")
    assert not is_decoder_projection("visual.layers.3.self_attn.q_proj.weight") and not is_decoder_projection("lm_head.weight")

    good = load_file(str(tmp_path / "w8" / "model.safetensors"))
    q = "model.layers.1.self_attn.k_proj.weight"

    def variant(name, edit, index=None):
        d = tmp_path / name
        d.mkdir()
        t = dict(good)
        edit(t)
        save_file({k: v.contiguous() for k, v in t.items()}, str(d / "model.safetensors"), metadata={"format": "pt"})
        if index is not None:
            (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": index(t)}))
        return d

    d = variant("float_proj", lambda t: (t.__setitem__(q, sd[q]), t.pop(q + "_scale")))
    with pytest.raises(TypeError, match="k_proj.weight' must be int8, got F16"):
        inspect_w8a16_checkpoint(d)
    # even when floating projections are tolerated, layers that differ in what they quantise are refused
    with pytest.raises(KeyError, match="different numbers of int8"):
        inspect_w8a16_checkpoint(d, require_all=False)
    d = variant("all_float", lambda t: [(t.__setitem__(n, t[n].half()), t.pop(n + "_scale")) for n in list(t)
                                        if n.endswith("proj.weight")])
    assert len(inspect_w8a16_checkpoint(d, require_all=False)["unquantized"]) == 7 * cfg.num_layers
    with pytest.raises(KeyError, match="has no 'model.layers.1.self_attn.k_proj.weight_scale'"):
        inspect_w8a16_checkpoint(variant("no_scale", lambda t: t.pop(q + "_scale")))
    with pytest.raises(KeyError, match="unexpected scale 'model.norm.weight_scale'"):
        inspect_w8a16_checkpoint(variant("stray_scale", lambda t: t.__setitem__("model.norm.weight_scale", torch.ones(4).half())))
    with pytest.raises(TypeError, match="must be fp16, got F32"):
        inspect_w8a16_checkpoint(variant("f32_scale", lambda t: t.__setitem__(q + "_scale", t[q + "_scale"].float())))
    with pytest.raises(ValueError, match="has shape"):
        inspect_w8a16_checkpoint(variant("short_scale", lambda t: t.__setitem__(q + "_scale", t[q + "_scale"][:-1])))
    with pytest.raises(TypeError, match="not a decoder projection"):
        inspect_w8a16_checkpoint(variant("int8_embed", lambda t: (t.__setitem__("model.embed_tokens.weight", t[q].clone()),
                                                                   t.__setitem__("model.embed_tokens.weight_scale", t[q + "_scale"].clone()))))
    with pytest.raises(TypeError, match="must be floating, got I64"):
        inspect_w8a16_checkpoint(variant("int_buffer", lambda t: t.__setitem__("model.position_ids", torch.arange(4))))
    d = variant("int_buffer_ok", lambda t: t.__setitem__("model.position_ids", torch.arange(4)))
    assert "model.position_ids" in inspect_w8a16_checkpoint(d, allow_integer=["model.position_ids"])["nondecoder"]
    with pytest.raises(KeyError, match="only in index \\['ghost.weight'\\]"):
        inspect_w8a16_checkpoint(variant("ghost", lambda t: None,
                                         index=lambda t: {**{n: "model.safetensors" for n in t}, "ghost.weight": "model.safetensors"}))
    lm = variant("int8_head", lambda t: (t.__setitem__("lm_head.weight", t[q].clone()),
                                         t.__setitem__("lm_head.weight_scale", t[q + "_scale"].clone())),
                 index=lambda t: {n: "model.safetensors" for n in t})
    with pytest.raises(TypeError, match="not a decoder projection"):
        inspect_w8a16_checkpoint(lm)
    assert "lm_head.weight" in inspect_w8a16_checkpoint(lm, extra_int8=["lm_head.weight"])["int8"]

    # two shards: a duplicate tensor and an index that points to the wrong shard
    two = tmp_path / "two"
    two.mkdir()
    names = sorted(good)
    a, b = {n: good[n] for n in names[::2]}, {n: good[n] for n in names[1::2]}
    save_file(a, str(two / "model-00001-of-00002.safetensors"), metadata={"format": "pt"})
    save_file(b, str(two / "model-00002-of-00002.safetensors"), metadata={"format": "pt"})
    wm = {**{n: "model-00001-of-00002.safetensors" for n in a}, **{n: "model-00002-of-00002.safetensors" for n in b}}
    (two / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    assert len(set(inspect_w8a16_checkpoint(two)["tensor_shards"].values())) == 2
    wrong = dict(wm)
    wrong[names[0]] = "model-00002-of-00002.safetensors"
    (two / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wrong}))
    with pytest.raises(KeyError, match="wrong shard"):
        inspect_w8a16_checkpoint(two)
    (two / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    save_file({**b, names[0]: good[names[0]]}, str(two / "model-00002-of-00002.safetensors"), metadata={"format": "pt"})
    with pytest.raises(KeyError, match="appears more than once"):
        inspect_w8a16_checkpoint(two)


def test_qwen3_vl_32b_w8a16_profile_predicate():
    import copy
    from types import SimpleNamespace
    from rpu_backend.quant.load import QWEN3_VL_32B_W8A16 as P, is_qwen3_vl_32b_w8a16_config
    base = {"architectures": ["Qwen3VLForConditionalGeneration"], **P["top"], "quant_config": dict(P["quant_config"]),
            "text_config": dict(P["text_config"]), "vision_config": dict(P["vision_config"])}
    assert is_qwen3_vl_32b_w8a16_config(base)
    as_object = SimpleNamespace(**{**base, "text_config": SimpleNamespace(**base["text_config"]),
                                   "vision_config": SimpleNamespace(**{**base["vision_config"],
                                                                       "deepstack_visual_indexes": (8, 16, 24)})})
    assert is_qwen3_vl_32b_w8a16_config(as_object)
    for path, value in ((("text_config", "num_hidden_layers"), 36), (("vision_config", "depth"), 24),
                        (("quant_config", "quantized_lm_head"), True), (("tie_word_embeddings",), True),
                        (("architectures",), ["Qwen3VLMoeForConditionalGeneration"]), (("text_config",), None),
                        (("vision_config", "deepstack_visual_indexes"), [8, 16]), (("text_config", "rms_norm_eps"), 1e-5),
                        (("quant_config", "extra"), 1)):
        c = copy.deepcopy(base)
        target = c
        for k in path[:-1]:
            target = target[k]
        target[path[-1]] = value
        assert not is_qwen3_vl_32b_w8a16_config(c), path
    assert not is_qwen3_vl_32b_w8a16_config({}) and not is_qwen3_vl_32b_w8a16_config(SimpleNamespace())
