"""Raw observation -> model inputs for Hy-Embodied-0.5-VLA (reference behaviour:
``python/rpu_backend/adapters/hy_vla/preprocess.py:40-377``).

The numbers below are those of the supported checkpoint's ``config.json``: three cameras in the order
:data:`CAMERA_ORDER`, frames letter-boxed to 224 x 224, a 7 x 7 patch grid per image after the merger, a 64-token prompt,
32-wide state and action vectors, 50 action steps, no placeholder for a missing camera (the prefix simply gets shorter),
``visual_segment_isolation = False``.

Prefix rows, in order::

    <bos> <user>                                                  2 rows
    per image:  <vision_start>  7 x (7 patches + 1 row split)  <vision_end>        1 + 56 + 1 = 58 rows
    prompt tokens, right-padded to 64                             64 rows

so three images give 2 + 3 * 58 + 64 = 240 rows whatever the prompt's real length; the consumer slices to its own
prefix length.  Only prompt padding is ever masked out.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

CAMERA_ORDER = ("observation.images.top_head", "observation.images.hand_left", "observation.images.hand_right")
ASSISTANT_TAG = "<｜hy_Assistant｜>"
LEAD_ROWS = 2
Range = Tuple[int, int]


# ----------------------------------------------------------------------------------------------------------- images
def resize_with_pad(img: torch.Tensor, width: int, height: int, pad_value: float = 0.0,
                    mode: str = "bilinear") -> torch.Tensor:
    """Scale ``[B, C, H, W]`` to fit inside ``height x width`` keeping the aspect ratio, then centre it.

    The scaled size is truncated, not rounded, and an odd amount of padding puts the extra row / column at the bottom /
    right: 480 x 640 becomes 168 x 224 with 28 rows above and below.  The patch grid depends on exactly this placement."""
    if img.ndim != 4:
        raise ValueError(f"expected (b, c, h, w), got {tuple(img.shape)}")
    h, w = img.shape[2:]
    shrink = max(w / width, h / height)
    new_h, new_w = int(h / shrink), int(w / shrink)
    kw = {} if mode == "nearest" else {"align_corners": False}
    scaled = F.interpolate(img, size=(new_h, new_w), mode=mode, **kw)
    extra_h, extra_w = max(0, height - new_h), max(0, width - new_w)
    top, left = extra_h // 2, extra_w // 2
    return F.pad(scaled, (left, extra_w - left, top, extra_h - top), value=pad_value)


def _frame_to_unit_nchw(frame: Any, cam: int) -> torch.Tensor:
    """One camera frame in any common form -> ``[1, 3, H, W]`` fp32 in [0, 1].

    Accepted: tensors or numpy arrays shaped ``[3,H,W]``, ``[1,3,H,W]``, ``[H,W,3]``, ``[1,H,W,3]`` (channel-first wins
    when both readings fit), and anything with ``.convert("RGB")`` (PIL).  Integer pixels are 0..255 and are divided;
    floating pixels must already be in [0, 1] - a float frame outside that range is refused rather than guessed at,
    because it could equally be an un-normalised 0..255 image or an already centred [-1, 1] model input.  Channel order
    is taken as RGB."""
    import numpy as np
    x = frame
    if not torch.is_tensor(x) and not isinstance(x, np.ndarray):
        if not hasattr(x, "convert"):
            raise TypeError(f"camera {cam}: unsupported frame type {type(x).__name__}; pass a torch.Tensor, a "
                            "numpy.ndarray or a PIL image")
        x = np.array(x.convert("RGB"))
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    if x.ndim == 3:
        x = x.unsqueeze(0)
    elif x.ndim != 4:
        raise ValueError(f"camera {cam}: a frame has 3 or 4 dimensions, got {tuple(x.shape)}")
    elif x.shape[0] != 1:
        raise ValueError(f"camera {cam}: one frame per camera, got a batch of {x.shape[0]}")
    if x.shape[1] != 3:
        if x.shape[-1] != 3:
            raise ValueError(f"camera {cam}: need 3 RGB channels, got {tuple(x.shape)}")
        x = x.permute(0, 3, 1, 2).contiguous()
    if x.dtype == torch.bool:
        raise ValueError(f"camera {cam}: a bool frame has no pixel interpretation")
    if not x.is_floating_point():
        return x.float() / 255.0
    x = x.float()
    lo, hi = (float(v) for v in torch.aminmax(x))
    if hi > 1.5 or lo < -0.01:
        raise ValueError(f"camera {cam}: float pixels span [{lo:.4g}, {hi:.4g}], not [0, 1]; divide 0..255 floats by 255 "
                         "before passing them (integer frames are divided automatically)")
    return x


def prepare_images(frames: Sequence[Any], size: int = 224) -> List[torch.Tensor]:
    """One frame per camera -> ``[1, 3, size, size]`` in [-1, 1]; the letter-box bars therefore hold -1."""
    return [resize_with_pad(_frame_to_unit_nchw(f, i), size, size, pad_value=0.0) * 2.0 - 1.0
            for i, f in enumerate(frames)]


# ----------------------------------------------------------------------------------------------- language and state
def prepare_language(instruction: str, tokenizer, max_length: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Instruction -> ``(tokens [1, L] int64, mask [1, L] bool)``, right-padded, without special tokens (the model adds
    its own BOS row).

    Underscores and newlines become spaces and the text is closed with the assistant tag.  The tag itself contains an
    underscore, so a caller-supplied trailing tag is removed before the clean-up and put back after it; bare and tagged
    instructions tokenise identically."""
    text = instruction.strip()
    if text.endswith(ASSISTANT_TAG):
        text = text[:-len(ASSISTANT_TAG)].strip()
    text = text.replace("_", " ").replace("\n", " ") + ASSISTANT_TAG
    enc = tokenizer([text], padding="max_length", padding_side="right", truncation=True, max_length=max_length,
                    return_tensors="pt", add_special_tokens=False)
    return enc["input_ids"].long(), enc["attention_mask"].bool()


def prepare_state(state: Any = None, max_state_dim: int = 32) -> torch.Tensor:
    """Proprioception -> ``[1, max_state_dim]`` fp32, zero-padded on the right; ``None`` is the zero state."""
    out = torch.zeros(1, max_state_dim)
    if state is not None:
        s = torch.as_tensor(state, dtype=torch.float32).reshape(1, -1)
        if s.shape[1] > max_state_dim:
            raise ValueError(f"state has {s.shape[1]} entries, more than max_state_dim={max_state_dim}")
        out[:, :s.shape[1]] = s
    return out


# ------------------------------------------------------------------------------------------------------------ masks
def make_att_2d_masks(pad_masks: torch.Tensor, att_masks: torch.Tensor) -> torch.Tensor:
    """Block-causal visibility from a 1-D block marker: a row sees the columns whose running sum of ``att_masks`` does
    not exceed its own, and only where both row and column are real (``pad_masks``).  All ones is plain causal;
    ``[1, 0, 0, ...]`` is one fully connected block."""
    if pad_masks.ndim != 2 or att_masks.ndim != 2:
        raise ValueError("pad_masks and att_masks are [batch, rows]")
    block = torch.cumsum(att_masks.long(), dim=1)
    real = pad_masks.bool()
    return (block[:, None, :] <= block[:, :, None]) & real[:, None, :] & real[:, :, None]


@dataclass(frozen=True)
class PrefixLayout:
    """Row arithmetic of the prefix for ``n_images`` images of ``grid x grid`` merged patches and ``n_lang`` prompt rows."""

    n_images: int
    grid: int
    n_lang: int

    @property
    def rows_per_image(self) -> int:
        return 1 + self.grid * (self.grid + 1) + 1

    @property
    def total(self) -> int:
        return LEAD_ROWS + self.n_images * self.rows_per_image + self.n_lang

    def image_body(self, i: int) -> Range:
        """Patches and row splits of image ``i``, without its start / end markers."""
        start = LEAD_ROWS + i * self.rows_per_image + 1
        return start, start + self.grid * (self.grid + 1)

    def patch_rows(self, i: int) -> List[Range]:
        """``[start, end)`` of each of the ``grid`` patch runs of image ``i`` (the split after each run excluded)."""
        s, _ = self.image_body(i)
        return [(s + r * (self.grid + 1), s + r * (self.grid + 1) + self.grid) for r in range(self.grid)]

    def image_id(self) -> torch.Tensor:
        """``[total]`` int64: the image a row's *patch* belongs to, -1 for every other row."""
        ids = torch.full((self.total,), -1, dtype=torch.long)
        for i in range(self.n_images):
            for s, e in self.patch_rows(i):
                ids[s:e] = i
        return ids


def prefix_masks(n_images: int, grid: int, lang_masks: torch.Tensor):
    """``(pad_masks, att_masks, modality_mask, image_idx_ranges, image_full_ranges)``; the masks are ``[1, rows]`` bool.

    Every row starts its own causal block (``att_masks`` all ones); ``modality_mask`` marks patch rows, which go through
    the visual weights; only prompt padding is False in ``pad_masks``."""
    lay = PrefixLayout(n_images, grid, int(lang_masks.shape[1]))
    pad = torch.ones(1, lay.total, dtype=torch.bool)
    pad[:, lay.total - lay.n_lang:] = lang_masks.bool()
    att = torch.ones(1, lay.total, dtype=torch.bool)
    modality = (lay.image_id() >= 0)[None]
    idx = [r for i in range(n_images) for r in lay.patch_rows(i)]
    full = [lay.image_body(i) for i in range(n_images)]
    return pad, att, modality, idx, full


def apply_visual_segment_mask(att_2d: torch.Tensor, image_idx_ranges: Sequence[Range],
                              image_full_ranges: Sequence[Range], isolation: bool = False) -> None:
    """In place: patches of one image see each other in both directions, patches of different images do not see each
    other at all; markers and row splits stay causal.  ``isolation=True`` (whole segments isolated) changes the numerics
    and is not supported."""
    if isolation:
        raise NotImplementedError("visual_segment_isolation=True is not supported; the supported checkpoint uses False")
    owner = torch.full((att_2d.shape[-1],), -1, dtype=torch.long)
    for img, (lo, hi) in enumerate(image_full_ranges):
        for s, e in image_idx_ranges:
            if lo <= s and e <= hi:
                owner[s:e] = img
    is_patch = owner >= 0
    among_patches = is_patch[:, None] & is_patch[None, :]
    same_image = among_patches & (owner[:, None] == owner[None, :])
    att_2d[:, among_patches] = False
    att_2d[:, same_image] = True


def suffix_masks(n_action: int = 50, n_state_tokens: int = 1):
    """Suffix = state token(s) then the action chunk: two blocks, each fully connected inside, causal between them.
    Returns ``(pad_masks, att_masks, modality_mask)``, all ``[1, n_state_tokens + n_action]``; every suffix row runs
    through the visual-side weights."""
    n = n_state_tokens + n_action
    att = torch.zeros(1, n, dtype=torch.bool)
    att[0, 0] = att[0, n_state_tokens] = True
    return torch.ones(1, n, dtype=torch.bool), att, torch.ones(1, n, dtype=torch.bool)


def sample_noise(n_action: int = 50, action_dim: int = 32, seed: Optional[int] = None) -> torch.Tensor:
    """Initial flow-matching sample ``[1, n_action, action_dim]`` fp32.  With a seed it comes from a private generator
    (reproducible, global RNG untouched); without, from the global RNG."""
    gen = None if seed is None else torch.Generator().manual_seed(int(seed))
    return torch.randn(1, n_action, action_dim, generator=gen, dtype=torch.float32)


# ------------------------------------------------------------------------------------------------------ observation
def build_observation(frames: Sequence[Any], instruction: str, tokenizer, *, state: Any = None,
                      noise: Optional[torch.Tensor] = None, noise_seed: Optional[int] = None, grid: int = 7,
                      max_state_dim: int = 32, max_action_dim: int = 32, n_action: int = 50,
                      tokenizer_max_length: int = 64, image_size: int = 224) -> Dict[str, Any]:
    """Everything the runner's ``get_action`` takes, plus ``n_valid`` (real prefix rows: the caller checks that it fits
    the prefix length the runner was built for instead of letting a long prompt be cut silently).

    ``denoise_mask`` is ``[suffix rows, prefix rows + suffix rows]``: every suffix row sees all real prefix rows, and the
    suffix block structure among themselves.  Suffix positions continue from the number of *real* prefix rows."""
    images = prepare_images(frames, size=image_size)
    tokens, lang_mask = prepare_language(instruction, tokenizer, max_length=tokenizer_max_length)
    pad_p, att_p, mod_p, idx, full = prefix_masks(len(images), grid, lang_mask)
    prefill_mask = make_att_2d_masks(pad_p, att_p)
    apply_visual_segment_mask(prefill_mask, idx, full)
    n_valid = int(pad_p.sum())
    pad_s, att_s, _ = suffix_masks(n_action)
    denoise_mask = torch.cat([pad_p[:, None, :].expand(1, pad_s.shape[1], pad_p.shape[1]),
                              make_att_2d_masks(pad_s, att_s)], dim=2)
    return {
        "images": images,
        "lang_tokens": tokens[0],
        "prefill_mask": prefill_mask[0],
        "prefill_pos": (torch.cumsum(pad_p.long(), dim=1) - 1)[0],
        "modality_mask": mod_p[0],
        "denoise_mask": denoise_mask[0],
        "suffix_pos": (n_valid + torch.cumsum(pad_s.long(), dim=1) - 1)[0],
        "noise": (sample_noise(n_action, max_action_dim, seed=noise_seed) if noise is None else noise).float(),
        "state": prepare_state(state, max_state_dim),
        "n_valid": n_valid,
    }


__all__ = ["CAMERA_ORDER", "ASSISTANT_TAG", "PrefixLayout", "resize_with_pad", "prepare_images", "prepare_language",
           "prepare_state", "make_att_2d_masks", "prefix_masks", "apply_visual_segment_mask", "suffix_masks",
           "sample_noise", "build_observation"]
