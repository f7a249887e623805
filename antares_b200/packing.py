"""Host-side int4 packing, seeded synthetic weights and tensor-parallel sharding (numpy; runs once
at load time, never on the per-token path).

Packed layout = the GPTQ checkpoint layout the reference sample consumes
(samples/05_llama2_7b_int4.py:24-28,136): qweight int32 [K/8, N], word (r, n) holds rows 8r..8r+7 of
column n, lowest nibble = lowest row; scales [K/group, N]; zero-point fixed at 8 (the sample drops
`qzeros`, lines 34-40) and no act-order (`g_idx` dropped, lines 52-58).
"""
import numpy as np

GROUP = 128


def pack_w4(q):
    """uint4 values [K, N] (any integer dtype, 0..15) -> int32 [K/8, N]."""
    q = np.asarray(q)
    K, N = q.shape
    if K % 8:
        raise ValueError("K=%d is not a multiple of 8" % K)
    if q.min() < 0 or q.max() > 15:
        raise ValueError("values outside 0..15")
    q = q.astype(np.uint32).reshape(K // 8, 8, N)
    w = np.zeros((K // 8, N), np.uint32)
    for j in range(8):
        w |= q[:, j, :] << np.uint32(4 * j)
    return w.view(np.int32)


def unpack_w4(qweight):
    """int32 [K/8, N] -> uint8 [K, N]."""
    qweight = np.ascontiguousarray(qweight, np.int32).view(np.uint32)
    Kp, N = qweight.shape
    out = np.empty((Kp, 8, N), np.uint8)
    for j in range(8):
        out[:, j, :] = (qweight >> np.uint32(4 * j)) & np.uint32(15)
    return out.reshape(Kp * 8, N)


def synth_w4(K, N, seed, group=GROUP, scales_dtype=np.float16, centered=False, scale_mul=1.0):
    """Seeded stand-in for a GPTQ layer: nibbles uniform in 0..15 (drawn as uniform 32-bit words),
    scales uniform in [0.001, 0.02].  centered=True turns every nibble 0 into an 8, so that q - 8 has
    zero mean, and scale_mul shrinks the scales (both used by tests that need a model whose layers add
    no common offset and do not amplify rounding differences)."""
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint32)
    if centered:
        for j in range(8):
            zero = ((w >> np.uint32(4 * j)) & np.uint32(15)) == 0
            w |= zero.astype(np.uint32) << np.uint32(4 * j + 3)
    qweight = w.view(np.int32)
    scales = rng.random((K // group, N), dtype=np.float32) * np.float32(0.019) + np.float32(0.001)
    if scale_mul != 1.0:
        scales *= np.float32(scale_mul)
    scales = scales.astype(scales_dtype)
    return qweight, scales


def synth_x(M, K, seed, dtype=np.float16):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((M, K), dtype=np.float32).astype(dtype)


# ---- tensor-parallel sharding (Megatron style) -----------------------------------------------------

def shard_columns(qweight, scales, rank, world):
    """Column-parallel slice: columns [rank*N/world, (rank+1)*N/world)."""
    N = qweight.shape[1]
    if N % (4 * world):
        raise ValueError("N=%d cannot be split into %d column shards of a multiple of 4" % (N, world))
    n = N // world
    sl = slice(rank * n, (rank + 1) * n)
    return np.ascontiguousarray(qweight[:, sl]), np.ascontiguousarray(scales[:, sl])


def row_shard_bounds(K, world, group=GROUP):
    """K ranges of a row-parallel split aligned to quantisation groups; shards may differ by one
    group when K/group is not a multiple of world (11008/128 = 86 groups over 4 or 8 ranks)."""
    groups = K // group
    bounds = [(groups * r) // world * group for r in range(world + 1)]
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def shard_rows(qweight, scales, rank, world, group=GROUP):
    """Row-parallel slice of K, group aligned: returns (qweight_r, scales_r, (k0, k1))."""
    K = qweight.shape[0] * 8
    k0, k1 = row_shard_bounds(K, world, group)[rank]
    return (np.ascontiguousarray(qweight[k0 // 8:k1 // 8]), np.ascontiguousarray(scales[k0 // group:k1 // group]), (k0, k1))


def tile_weights(qweight, scales, tile=128):
    """Reference layout qweight [K/8, N], scales [K/group, N] -> tile-major [N/tile][K/8][tile],
    [N/tile][K/group][tile] (numpy), the layout ab200_w4a16_gemv_tiled streams."""
    qweight, scales = np.asarray(qweight), np.asarray(scales)
    n = qweight.shape[1]
    if n % tile:
        raise ValueError("N=%d is not a multiple of %d" % (n, tile))
    q = np.ascontiguousarray(qweight.reshape(qweight.shape[0], n // tile, tile).transpose(1, 0, 2))
    s = np.ascontiguousarray(scales.reshape(scales.shape[0], n // tile, tile).transpose(1, 0, 2))
    return q, s
