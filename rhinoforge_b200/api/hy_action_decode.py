"""Hy-Embodied VLA action contract: raw end-effector pose -> model state, and model action chunk -> physical poses.

The model emits, per arm, ``[dx, dy, dz, r6, gripper]`` relative to the pose *at the start of the chunk* (not chained),
where ``r6`` is the 6-D rotation parameterisation: the first two **rows** of the relative rotation matrix, completed by
Gram-Schmidt.  Decoding de-normalises the chunk with the per-step statistics of the checkpoint, composes every step with
the start pose (``R = R0 dR``, ``t = t0 + R0 dt``) and returns ``[x, y, z, quaternion, gripper]`` per arm.  Both
directions live in one object because they share the statistics and the coordinate-frame switches; configuring only one
of them yields a trajectory that is self-consistent and wrong.  Reference behaviour:
``python/rpu_backend/api/hy_action_decode.py:40-258``.

Layouts: a dual-arm pose is 16 wide, ``[l_xyz 3, l_quat 4, l_grip 1, r_xyz 3, r_quat 4, r_grip 1]``; a dual-arm action
is 20 wide, ``[l_t 3, l_r6 6, l_grip 1, r_t 3, r_r6 6, r_grip 1]``.  Quaternions are ``xyzw`` inside this module and
``wxyz`` at the :class:`HyVlaActionDecoder` interface.  Checkpoints trained on UMI data use another world frame and
another tool-axis order: ``p_umi = W p``, ``R_umi = W R P``; with ``umi_gripper_space`` the gripper also changes from
1 = open / 0 = closed to millimetres, 0 = open / 90 = closed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import numpy as np

ARM_DIMS = 10          # 3 translation + 6 rotation + 1 gripper
POSE_DIMS = 8          # 3 position + 4 quaternion + 1 gripper
WORLD_TO_UMI = np.array([[0, 1, 0], [-1, 0, 0], [0, 0, 1]], dtype=np.float64)       # W
TOOL_AXES_TO_UMI = np.array([[0, 0, 1], [1, 0, 0], [0, 1, 0]], dtype=np.float64)    # P (a column permutation)
GRIPPER_CLOSED_MM = 90.0


# ----------------------------------------------------------------------------------------------------- rotations
def rotation_6d_to_matrix(d6: np.ndarray) -> np.ndarray:
    """``[..., 6]`` -> ``[..., 3, 3]``: the two encoded vectors are orthonormalised into rows 0 and 1, row 2 is their
    cross product."""
    d6 = np.asarray(d6, dtype=np.float64)
    a1, a2 = d6[..., :3], d6[..., 3:6]
    b1 = a1 / np.maximum(np.linalg.norm(a1, axis=-1, keepdims=True), 1e-12)
    a2 = a2 - (b1 * a2).sum(-1, keepdims=True) * b1
    b2 = a2 / np.maximum(np.linalg.norm(a2, axis=-1, keepdims=True), 1e-12)
    return np.stack((b1, b2, np.cross(b1, b2)), axis=-2)


def matrix_to_rotation_6d(m: np.ndarray) -> np.ndarray:
    """``[..., 3, 3]`` -> ``[..., 6]``: rows 0 and 1."""
    m = np.asarray(m, dtype=np.float64)
    return np.concatenate((m[..., 0, :], m[..., 1, :]), axis=-1)


def quat_xyzw_to_matrix(q: np.ndarray) -> np.ndarray:
    q = np.asarray(q, dtype=np.float64)
    x, y, z, w = (q[..., i] for i in range(4))
    n = np.maximum(np.sqrt(x * x + y * y + z * z + w * w), 1e-12)
    x, y, z, w = x / n, y / n, z / n, w / n
    return np.stack((np.stack((1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)), -1),
                     np.stack((2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)), -1),
                     np.stack((2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)), -1)), -2)


def matrix_to_quat_xyzw(m: np.ndarray) -> np.ndarray:
    m = np.asarray(m, dtype=np.float64)
    out = np.empty(m.shape[:-2] + (4,), dtype=np.float64)
    flat_m, flat_o = m.reshape(-1, 3, 3), out.reshape(-1, 4)
    for i, r in enumerate(flat_m):
        t = np.trace(r)
        if t > 0:
            s = np.sqrt(t + 1.0) * 2
            q = ((r[2, 1] - r[1, 2]) / s, (r[0, 2] - r[2, 0]) / s, (r[1, 0] - r[0, 1]) / s, 0.25 * s)
        else:
            k = int(np.argmax(np.diag(r)))
            a, b = (k + 1) % 3, (k + 2) % 3
            s = np.sqrt(1.0 + r[k, k] - r[a, a] - r[b, b]) * 2
            v = [0.0, 0.0, 0.0, 0.0]
            v[k], v[a], v[b], v[3] = 0.25 * s, (r[a, k] + r[k, a]) / s, (r[b, k] + r[k, b]) / s, (r[b, a] - r[a, b]) / s
            q = tuple(v)
        flat_o[i] = q
    return out


# --------------------------------------------------------------------------------------------- relative -> absolute
def relative_to_absolute_poses(rel: np.ndarray, start_xyzw: np.ndarray) -> np.ndarray:
    """One arm: ``rel [H, 10]`` + start ``[x, y, z, qx, qy, qz, qw]`` -> ``[H, 8]`` = pose (xyzw) + gripper.  The
    gripper takes no part in the composition and passes through."""
    rel = np.asarray(rel, dtype=np.float64)
    start = np.asarray(start_xyzw, dtype=np.float64)
    R0, t0 = quat_xyzw_to_matrix(start[3:7]), start[:3]
    R = R0[None] @ rotation_6d_to_matrix(rel[:, 3:9])
    t = t0[None] + rel[:, :3] @ R0.T
    return np.concatenate((t, matrix_to_quat_xyzw(R), rel[:, 9:10]), axis=1)


def relative_to_dual_arm_poses(rel20: np.ndarray, start_dual_xyzw: np.ndarray) -> np.ndarray:
    """``[H, 20]`` + the 16-wide start pose (a 14-wide one without grippers is accepted too) -> ``[H, 16]``."""
    rel20 = np.asarray(rel20, dtype=np.float64)
    start = np.asarray(start_dual_xyzw, dtype=np.float64).reshape(-1)
    if start.shape[0] not in (14, 16):
        raise ValueError(f"dual-arm start pose is 16 wide (14 without grippers), got {start.shape[0]}")
    right_at = 8 if start.shape[0] == 16 else 7
    left = relative_to_absolute_poses(rel20[:, :ARM_DIMS], start[:7])
    right = relative_to_absolute_poses(rel20[:, ARM_DIMS:2 * ARM_DIMS], start[right_at:right_at + 7])
    return np.concatenate((left, right), axis=1)


# ------------------------------------------------------------------------------------------------ frames, layouts
def _per_arm(a: np.ndarray):
    """Views ``(position, quaternion, gripper index)`` of both arms in a ``[N, 16]`` array."""
    return ((a[:, 0:3], a[:, 3:7], 7), (a[:, 8:11], a[:, 11:15], 15))


def convert_frame(pose16_xyzw: np.ndarray, *, to_umi: bool, convert_gripper: bool = False) -> np.ndarray:
    """Native world / tool frame <-> UMI frame for ``[N, 16]`` dual-arm poses (xyzw)."""
    out = np.array(pose16_xyzw, dtype=np.float64, copy=True)
    if out.shape[0] == 0:
        return out
    W, P = (WORLD_TO_UMI, TOOL_AXES_TO_UMI) if to_umi else (WORLD_TO_UMI.T, TOOL_AXES_TO_UMI.T)
    for pos, quat, grip in _per_arm(out):
        pos[:] = pos @ W.T
        quat[:] = matrix_to_quat_xyzw(W @ quat_xyzw_to_matrix(quat) @ P)
        if convert_gripper:
            out[:, grip] = (1.0 - out[:, grip]) * GRIPPER_CLOSED_MM if to_umi else 1.0 - out[:, grip] / GRIPPER_CLOSED_MM
    return out


def _swap_quat(a: np.ndarray, order) -> np.ndarray:
    out = np.array(a, dtype=np.float64, copy=True)
    for base in (3, 11):
        out[..., base:base + 4] = np.asarray(a, dtype=np.float64)[..., [base + k for k in order]]
    return out


def quat_wxyz_to_xyzw(pose16: np.ndarray) -> np.ndarray:
    return _swap_quat(pose16, (1, 2, 3, 0))


def quat_xyzw_to_wxyz(pose16: np.ndarray) -> np.ndarray:
    return _swap_quat(pose16, (3, 0, 1, 2))


def pose_to_rot6d(pose16_xyzw: np.ndarray) -> np.ndarray:
    """``[N, 16]`` position + quaternion -> ``[N, 20]`` position + 6-D rotation (+ gripper), the state encoding."""
    p = np.asarray(pose16_xyzw, dtype=np.float64)
    out = np.zeros((p.shape[0], 2 * ARM_DIMS))
    for (pos, quat, grip), dst in zip(_per_arm(p), (0, ARM_DIMS)):
        out[:, dst:dst + 3] = pos
        out[:, dst + 3:dst + 9] = matrix_to_rotation_6d(quat_xyzw_to_matrix(quat))
        out[:, dst + 9] = p[:, grip]
    return out


# ------------------------------------------------------------------------------------------------------- decoder
@dataclass
class HyVlaActionDecoder:
    """The normalisation contract of one checkpoint.  Nothing about a robot is built in: the statistics come from the
    checkpoint's ``norm_stats`` and the frame switches from the caller - the defaults (UMI frame, native gripper
    units) are those of the released checkpoint and are not guaranteed to suit another robot."""

    act_mean: np.ndarray                       # [H, 20], per time step
    act_std: np.ndarray                        # [H, 20]
    qpos_mean: Optional[np.ndarray] = None     # [20], used by encode_state only
    qpos_std: Optional[np.ndarray] = None      # [20]
    umi_coord_frame: bool = True
    umi_gripper_space: bool = False
    drop_first: bool = True                    # the executed sequence is actions[1:]

    def __post_init__(self):
        self.act_mean, self.act_std = np.asarray(self.act_mean, np.float64), np.asarray(self.act_std, np.float64)
        if self.act_mean.shape != self.act_std.shape:
            raise ValueError(f"act_mean {self.act_mean.shape} and act_std {self.act_std.shape} differ in shape")
        if self.act_mean.ndim != 2 or self.act_mean.shape[1] != 2 * ARM_DIMS:
            raise ValueError(f"action statistics are [H, {2 * ARM_DIMS}], got {self.act_mean.shape}")
        if self.umi_gripper_space and not self.umi_coord_frame:
            raise ValueError("umi_gripper_space=True requires umi_coord_frame=True")

    @classmethod
    def from_norm_stats_mapping(cls, info: Mapping, *, source: str = "norm_stats", **kwargs) -> "HyVlaActionDecoder":
        """From the de-serialised statistics: ``action_mean`` / ``action_std`` are required, ``qpos_mean`` /
        ``qpos_std`` optional.  Statistics that also carry ``action_mean_abs`` / ``action_std_abs`` belong to a
        checkpoint trained with mixed absolute / relative actions, a decoding branch that is not implemented here and is
        refused rather than decoded as purely relative."""
        if not isinstance(info, Mapping):
            raise TypeError(f"{source} must de-serialise to a mapping, got {type(info).__name__}")
        for key in ("action_mean", "action_std"):
            if key not in info:
                raise KeyError(f"{source} lacks {key!r} (has: {sorted(info)})")
        if info.get("action_mean_abs") is not None and info.get("action_std_abs") is not None:
            raise NotImplementedError(f"{source} carries action_*_abs: the checkpoint mixes absolute and relative actions; "
                                      "only the purely relative form is implemented")
        opt = lambda k: None if info.get(k) is None else np.asarray(info[k], dtype=np.float64)
        return cls(np.asarray(info["action_mean"], np.float64), np.asarray(info["action_std"], np.float64),
                   opt("qpos_mean"), opt("qpos_std"), **kwargs)

    @property
    def horizon(self) -> int:
        return int(self.act_mean.shape[0])

    def encode_state(self, ee_pose16_wxyz) -> np.ndarray:
        """Current dual-arm pose ``[16]`` (wxyz) -> normalised model state ``[1, 20]``:
        wxyz -> xyzw, frame change, quaternion -> 6-D rotation, ``(x - mean) / (std + 1e-8)``."""
        if self.qpos_mean is None or self.qpos_std is None:
            raise ValueError("the statistics hold no qpos_mean / qpos_std: the state cannot be encoded")
        pose = quat_wxyz_to_xyzw(np.asarray(ee_pose16_wxyz, dtype=np.float64).reshape(-1)[:16])[None]
        if self.umi_coord_frame:
            pose = convert_frame(pose, to_umi=True, convert_gripper=self.umi_gripper_space)
        return (pose_to_rot6d(pose) - self.qpos_mean) / (self.qpos_std + 1e-8)

    def decode(self, actions_norm, initial_ee_pose_wxyz) -> np.ndarray:
        """``[H, >= 20]`` (or ``[1, H, .]``) normalised actions + the *current* dual-arm pose ``[16]`` (wxyz, the world
        frame of training) -> physical poses ``[H - 1, 16]`` (wxyz; ``[H, 16]`` with ``drop_first=False``).  Columns
        past 20 are padding.  A wrong start pose shifts the whole trajectory and raises nothing."""
        a = np.asarray(actions_norm, dtype=np.float64)
        if a.ndim == 3:
            if a.shape[0] != 1:
                raise ValueError(f"batch 1 only, got {a.shape}")
            a = a[0]
        if a.ndim != 2:
            raise ValueError(f"actions are [H, D], got {a.shape}")
        steps = a.shape[0]
        if steps > self.horizon:
            raise ValueError(f"{steps} action steps exceed the {self.horizon} steps of the statistics")
        if a.shape[1] < 2 * ARM_DIMS:
            raise ValueError(f"actions have {a.shape[1]} columns, at least {2 * ARM_DIMS} are needed")
        start = np.asarray(initial_ee_pose_wxyz, dtype=np.float64).reshape(-1)
        if start.shape[0] < 16:
            raise ValueError(f"initial_ee_pose needs 16 entries, got {start.shape[0]}")
        start = quat_wxyz_to_xyzw(start[:16])
        if self.umi_coord_frame:
            start = convert_frame(start[None], to_umi=True, convert_gripper=self.umi_gripper_space)[0]
        rel = a[:, :2 * ARM_DIMS] * self.act_std[:steps] + self.act_mean[:steps]
        poses = relative_to_dual_arm_poses(rel, start)
        if self.umi_coord_frame:
            poses = convert_frame(poses, to_umi=False, convert_gripper=self.umi_gripper_space)
        poses = quat_xyzw_to_wxyz(poses)
        return poses[1:] if self.drop_first else poses


__all__ = ["rotation_6d_to_matrix", "matrix_to_rotation_6d", "quat_xyzw_to_matrix", "matrix_to_quat_xyzw",
           "relative_to_absolute_poses", "relative_to_dual_arm_poses", "convert_frame", "quat_wxyz_to_xyzw",
           "quat_xyzw_to_wxyz", "pose_to_rot6d", "HyVlaActionDecoder", "ARM_DIMS", "POSE_DIMS"]
