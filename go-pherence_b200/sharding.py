"""Host-side partitioning for the multi-GPU forms: which rows of a projection and which experts
of a MoE layer a rank owns, and how to cut a rank's part out of the checkpoint arrays.

Rows are contiguous in every supported format (MLX words and group tables, GGUF blocks, FP8 bytes
are all row-major), so a rank's shard is a plain slice that goes through the ordinary upload entry
points.  The reference is single-GPU and has no counterpart."""
import numpy as np

Q8_0_BLOCK, Q4_K_BLOCK = (32, 34), (256, 144)   # (elements, bytes) per block; loader/gguf/quant_matrix.go:26-60
Q5_K_BLOCK, Q6_K_BLOCK = (256, 176), (256, 210)  # loader/gguf/quant_matrix.go:331-426


def shard_rows(out_dim, rank, world, align=8):
    """Rows [lo, hi) owned by `rank`: contiguous, cut at multiples of `align`; same rule as goph_shard_rows."""
    if out_dim < 0 or world <= 0 or not 0 <= rank < world or align <= 0:
        raise ValueError("bad shard request")
    blocks = (out_dim + align - 1) // align
    per = (blocks + world - 1) // world * align
    lo = min(out_dim, rank * per)
    return lo, min(out_dim, lo + per)


def slice_mlx(weight, scales, biases, in_dim, group_size, lo, hi):
    wpr, gpr = in_dim // 8, in_dim // group_size
    return (np.ascontiguousarray(weight[lo * wpr:hi * wpr]), np.ascontiguousarray(scales[lo * gpr:hi * gpr]),
            np.ascontiguousarray(biases[lo * gpr:hi * gpr]))


def slice_gguf(raw, block, in_dim, lo, hi):
    """block: Q8_0_BLOCK, Q4_K_BLOCK, Q5_K_BLOCK or Q6_K_BLOCK."""
    row_bytes = in_dim // block[0] * block[1]
    return np.ascontiguousarray(raw[lo * row_bytes:hi * row_bytes])


def slice_fp8(weight, scale, bias, in_dim, lo, hi):
    s = scale if len(scale) == 1 else np.ascontiguousarray(scale[lo:hi])
    b = None if bias is None else np.ascontiguousarray(bias[lo:hi])
    return np.ascontiguousarray(weight[lo * in_dim:hi * in_dim]), s, b


def place_experts(num_experts, rank, world):
    """Experts resident on `rank`: contiguous blocks (128 experts on 8 GPUs -> 16 each)."""
    per = (num_experts + world - 1) // world
    return range(min(num_experts, rank * per), min(num_experts, (rank + 1) * per))
