"""Data-only table of the built-in architecture adapters: (HF architecture, module, class).

Kept free of imports so that package start-up never loads a model module
(reference: ``python/rpu_backend/adapters/_manifest.py:10-41``)."""

BUILTIN_ADAPTERS = (
    ("Qwen3ForCausalLM", "rhinoforge_b200.adapters.qwen3", "Qwen3Adapter"),
    ("LlamaForCausalLM", "rhinoforge_b200.adapters.llama", "LlamaAdapter"),
    ("DINOv3ViTModel", "rhinoforge_b200.adapters.dinov3", "DINOv3Adapter"),
    ("SiglipVisionModel", "rhinoforge_b200.adapters.siglip", "SiglipAdapter"),
    ("Qwen3_5ForConditionalGeneration", "rhinoforge_b200.adapters.qwen3_5", "Qwen3_5Adapter"),
    ("Qwen3VLForConditionalGeneration", "rhinoforge_b200.adapters.qwen3_vl", "Qwen3VLAdapter"),
)

__all__ = ["BUILTIN_ADAPTERS"]
