"""Decoding of relative end-effector actions in the 6-D rotation parameterisation: each arm's action is
``[dx, dy, dz, r6 (two columns of the rotation), gripper]`` relative to the pose at the start of the chunk;
decoding turns a chunk into absolute ``[x, y, z, qx, qy, qz, qw, gripper]`` poses
(reference: ``python/rpu_backend/api/hy_action_decode.py:51-139``)."""
from __future__ import annotations

import numpy as np

ARM_DIMS = 10          # 3 translation + 6 rotation + 1 gripper


def rotation_6d_to_matrix(d6: np.ndarray) -> np.ndarray:
    """``[..., 6]`` -> ``[..., 3, 3]`` by Gram-Schmidt on the two encoded columns."""
    a1, a2 = d6[..., :3], d6[..., 3:6]
    b1 = a1 / np.maximum(np.linalg.norm(a1, axis=-1, keepdims=True), 1e-12)
    a2 = a2 - (b1 * a2).sum(-1, keepdims=True) * b1
    b2 = a2 / np.maximum(np.linalg.norm(a2, axis=-1, keepdims=True), 1e-12)
    b3 = np.cross(b1, b2)
    return np.stack((b1, b2, b3), axis=-1)


def quat_xyzw_to_matrix(q: np.ndarray) -> np.ndarray:
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


def relative_to_absolute_poses(rel: np.ndarray, start_xyzw: np.ndarray) -> np.ndarray:
    """``rel [H, 10]`` (one arm) + start pose ``[x,y,z,qx,qy,qz,qw]`` -> ``[H, 8]`` absolute poses + gripper.
    Every step is relative to the START pose (not chained): ``R = R0 * dR``, ``t = t0 + R0 * dt``."""
    rel = np.asarray(rel, dtype=np.float64)
    R0 = quat_xyzw_to_matrix(np.asarray(start_xyzw[3:7], dtype=np.float64))
    t0 = np.asarray(start_xyzw[:3], dtype=np.float64)
    dR = rotation_6d_to_matrix(rel[:, 3:9])
    R = R0[None] @ dR
    t = t0[None] + rel[:, :3] @ R0.T
    return np.concatenate((t, matrix_to_quat_xyzw(R), rel[:, 9:10]), axis=1)


def relative_to_dual_arm_poses(rel20: np.ndarray, start_dual_xyzw: np.ndarray) -> np.ndarray:
    """``[H, 20]`` (left arm | right arm) + ``[14]`` start poses -> ``[H, 16]``."""
    left = relative_to_absolute_poses(rel20[:, :ARM_DIMS], start_dual_xyzw[:7])
    right = relative_to_absolute_poses(rel20[:, ARM_DIMS:2 * ARM_DIMS], start_dual_xyzw[7:14])
    return np.concatenate((left, right), axis=1)


__all__ = ["rotation_6d_to_matrix", "quat_xyzw_to_matrix", "matrix_to_quat_xyzw", "relative_to_absolute_poses",
           "relative_to_dual_arm_poses", "ARM_DIMS"]
