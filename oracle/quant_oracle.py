"""CPU oracle for quantise / scale-pack / block-scaled GEMM.  TEST INFRASTRUCTURE ONLY.

The shipped package never imports this module; tests, the smoke check and the
benchmark's CPU-baseline leg use it as the checker for the CUDA path.

Pinning status
--------------
* GEMM algebra on already-quantised operands is pinned by golden vectors
  generated from the reference's own CPU emulation
  (tilelang/gemm/gemm_kernels.py:96-133, `fp8_gemm_tiled`, `grouped_gemm_tiled`)
  and by a C restatement of cuda/gemm/fp8_gemm.cu:29-99, cuda/gemm/fp4_gemm.cu:95-137
  and cuda/gemm/grouped_gemm.cu:79-104.
* FP8 per-tensor quantisation follows cuda/gemm/fp8_gemm.cu:119-144 and the
  "ref32" FP4 format follows cuda/gemm/fp4_gemm.cu:50-90; both are checked
  bit-for-bit against the C restatement of those kernels.
* NVFP4 (E4M3 scale per 16 + fp32 global scale), MXFP4 (E8M0 scale per 32),
  FP8 1x128 / 128x128 scaling and the swizzled scale-factor layout do not exist
  in the reference (its "NVFP4" and "MXFP4" are one fp32-scale-per-32 format,
  cuda/gemm/fp4_gemm.cu:30-42,107), so for those rules: PARITY UNPINNED - the
  rules below are this project's frozen definition, following the public
  format definitions.

All arithmetic is IEEE fp32 (numpy float32 ops are correctly rounded and never
contracted into FMAs).  Blocks run along the last (K) axis.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
U8 = np.uint8

# e2m1 decode table; order and values of cuda/gemm/fp4_gemm.cu:30-33
# (low nibble = even element, high nibble = odd element: fp4_gemm.cu:46,88).
E2M1_LUT = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=F32)

FP8_MAX = F32(448.0)
FP4_MAX = F32(6.0)
SCALE_FLOOR = F32(1e-12)       # fp8_gemm.cu:134, fp4_gemm.cu:70
FLT_MIN = F32(np.finfo(np.float32).tiny)


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x), dtype=F32)


# ----------------------------------------------------------------------------
# Code-point encoders / decoders (integer bit manipulation, no library casts)
# ----------------------------------------------------------------------------

def e4m3_encode(x) -> np.ndarray:
    """fp32 -> E4M3 byte: round-to-nearest-even, saturate to +-448, NaN -> 0x7F.

    Behaviour of `__nv_fp8_e4m3(float)` used at cuda/gemm/fp8_gemm.cu:142.
    """
    x = _f32(x)
    bits = x.view(np.uint32)
    sign = ((bits >> np.uint32(24)) & np.uint32(0x80)).astype(U8)
    nan = np.isnan(x)
    a = np.abs(np.where(nan, F32(0), x))
    a = np.minimum(a, FP8_MAX)
    ab = a.view(np.uint32)
    rounded = ab + np.uint32(0x7FFFF) + ((ab >> np.uint32(20)) & np.uint32(1))
    code_n = (rounded >> np.uint32(20)).astype(np.int64) - ((127 - 7) << 3)
    code_s = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)   # ties to even
    code = np.where(a < F32(2.0 ** -6), code_s, code_n)
    code = np.clip(code, 0, 0x7E)
    out = code.astype(U8) | sign
    return np.where(nan, U8(0x7F), out).astype(U8)


def _build_e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=F32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = float("nan")
        elif e == 0:
            v = s * m * 2.0 ** -9
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


E4M3_TABLE = _build_e4m3_table()


def e4m3_decode(b) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, dtype=U8)]


def e2m1_encode_rne(v) -> np.ndarray:
    """fp32 -> e2m1 nibble, round-to-nearest ties-to-even, saturating at +-6,
    sign bit copied from the input (so -0 is nibble 8).  Inputs must not be NaN."""
    v = _f32(v)
    sign = ((v.view(np.uint32) >> np.uint32(28)) & np.uint32(0x8)).astype(U8)
    a = np.abs(v)
    code = ((a > F32(0.25)).astype(U8) + (a >= F32(0.75)) + (a > F32(1.25))
            + (a >= F32(1.75)) + (a > F32(2.5)) + (a >= F32(3.5)) + (a > F32(5.0)))
    return (code.astype(U8) | sign).astype(U8)


def e2m1_encode_ref_lut(v) -> np.ndarray:
    """Nearest LUT entry by linear scan with strict '<' (first minimum wins, so
    ties go to the lower index): cuda/gemm/fp4_gemm.cu:80-87."""
    v = _f32(v)
    flat = v.reshape(-1)
    out = np.empty(flat.shape, dtype=U8)
    step = 1 << 18
    for s in range(0, flat.size, step):
        err = np.abs(E2M1_LUT[None, :] - flat[s:s + step, None])   # fp32, as the kernel
        out[s:s + step] = np.argmin(err, axis=1).astype(U8)
    return out.reshape(v.shape)


def e2m1_decode(n) -> np.ndarray:
    return E2M1_LUT[np.asarray(n, dtype=U8) & U8(0xF)]


def pack_nibbles(n: np.ndarray) -> np.ndarray:
    """[..., K] nibbles -> [..., K/2] bytes, low nibble = even k (fp4_gemm.cu:88)."""
    n = np.asarray(n, dtype=U8)
    assert n.shape[-1] % 2 == 0
    return (n[..., 0::2] | (n[..., 1::2] << U8(4))).astype(U8)


def unpack_nibbles(p: np.ndarray) -> np.ndarray:
    p = np.asarray(p, dtype=U8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=U8)
    out[..., 0::2] = p & U8(0xF)
    out[..., 1::2] = p >> U8(4)
    return out


def e8m0_decode(b) -> np.ndarray:
    """E8M0 byte -> 2^(b-127) as fp32 (0xFF is NaN and never produced here)."""
    e = np.asarray(b, dtype=np.int32) - 127
    return np.ldexp(F32(1.0), e).astype(F32)


# ----------------------------------------------------------------------------
# FP8 quantisers
# ----------------------------------------------------------------------------

def _fp8_scale(amax: np.ndarray) -> np.ndarray:
    s = (amax / FP8_MAX).astype(F32)                 # fp8_gemm.cu:133
    return np.maximum(s, SCALE_FLOOR).astype(F32)    # fp8_gemm.cu:134


def quant_fp8_per_tensor(x, scale=None):
    """cuda/gemm/fp8_gemm.cu:119-144: scale = max(amax/448, 1e-12), q = e4m3(x / scale).
    Returns (bytes like x, fp32 scalar)."""
    x = _f32(x)
    if scale is None:
        amax = np.max(np.abs(x)) if x.size else F32(0)
        s = _fp8_scale(np.asarray(amax, dtype=F32))
    else:
        s = np.asarray(scale, dtype=F32)
    q = e4m3_encode((x / s).astype(F32))             # division: fp8_gemm.cu:141
    return q, F32(s)


def quant_fp8_groupwise(x, group: int = 128):
    """1 x `group` scaling along K (scale layout of fp8_gemm.cu:74: [M, ceil(K/G)])."""
    x = _f32(x)
    M, K = x.shape
    ng = (K + group - 1) // group
    pad = ng * group - K
    xp = np.pad(x, ((0, 0), (0, pad))) if pad else x
    xg = xp.reshape(M, ng, group)
    s = _fp8_scale(np.max(np.abs(xg), axis=2))
    q = e4m3_encode((xg / s[:, :, None]).astype(F32)).reshape(M, ng * group)[:, :K]
    return np.ascontiguousarray(q), s


def quant_fp8_block(w, block: int = 128):
    """`block` x `block` scaling of a K-major weight [N, K]; scales [ceil(N/b), ceil(K/b)]."""
    w = _f32(w)
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = np.pad(w, ((0, nb * block - N), (0, kb * block - K)))
    wb = wp.reshape(nb, block, kb, block)
    s = _fp8_scale(np.max(np.abs(wb), axis=(1, 3)))
    q = e4m3_encode((wb / s[:, None, :, None]).astype(F32)).reshape(nb * block, kb * block)
    return np.ascontiguousarray(q[:N, :K]), s


# ----------------------------------------------------------------------------
# FP4 quantisers
# ----------------------------------------------------------------------------

def quant_fp4_ref32(x, tie: str = "ref_lut"):
    """The reference's only FP4 format (cuda/gemm/fp4_gemm.cu:50-90), over the FLAT
    buffer: per 32 contiguous elements scale = max(amax/6, 1e-12) (fp32),
    v = x * (1/scale), nearest e2m1.  Returns (packed bytes [n/2], scales [ceil(n/32)])."""
    flat = _f32(x).reshape(-1)
    n = flat.size
    nb = (n + 31) // 32
    xp = np.pad(flat, (0, nb * 32 - n)).reshape(nb, 32)
    amax = np.max(np.abs(xp), axis=1)
    s = np.maximum((amax / FP4_MAX).astype(F32), SCALE_FLOOR).astype(F32)
    inv = (F32(1.0) / s).astype(F32)
    v = (xp * inv[:, None]).astype(F32)
    enc = e2m1_encode_ref_lut if tie == "ref_lut" else e2m1_encode_rne
    nib = enc(v).reshape(-1)
    nib = nib[: n + (n & 1)]
    return pack_nibbles(nib), s


def nvfp4_global_scale(x) -> np.float32:
    x = _f32(x)
    amax = np.max(np.abs(x)) if x.size else F32(0)
    if amax == 0:
        return F32(1.0)
    return F32(F32(amax) / F32(448.0 * 6.0))


def nvfp4_token_scales(x) -> np.ndarray:
    """Per-token global scales: amax of each row / 2688 (1 for an all-zero row), fp32 [M]."""
    x = _f32(x)
    amax = np.max(np.abs(x), axis=1).astype(F32) if x.shape[1] else np.zeros(x.shape[0], F32)
    gs = (amax / F32(448.0 * 6.0)).astype(F32)
    return np.where(amax == 0, F32(1.0), gs).astype(F32)


def quant_nvfp4(x, global_scale=None):
    """NVFP4: e2m1 values, one unsigned-E4M3 scale per 16 K-elements, fp32 global scale.

    gs  = amax_tensor / 2688 (1 if the tensor is all zero) unless supplied
    sf  = ue4m3_rne(min((amax_16 / 6) / gs, 448))
    d   = f32(sf) * gs ;  inv = 1/d if d >= FLT_MIN else 0
    q   = e2m1_rne(x * inv)      (saturating at +-6)
    Returns (packed [M, K/2], sf bytes linear [M, K/16], gs).

    global_scale="per_token": the same rule with one global scale PER ROW, gs[m] = amax_row[m] / 2688 (1 for an
    all-zero row); gs is then an fp32 array [M].  A row's quantisation needs nothing but that row, so the quantiser
    is one pass over x; the product applies gs[m] as a per-token factor (see gemm_nvfp4)."""
    x = _f32(x)
    M, K = x.shape
    assert K % 16 == 0
    if isinstance(global_scale, str):
        if global_scale != "per_token":
            raise ValueError("global_scale must be None, a number or 'per_token'")
        gs = nvfp4_token_scales(x)
        gs_b = gs[:, None]
    else:
        gs = nvfp4_global_scale(x) if global_scale is None else F32(global_scale)
        gs_b = gs
    xb = x.reshape(M, K // 16, 16)
    amax = np.max(np.abs(xb), axis=2)
    t = ((amax / FP4_MAX).astype(F32) / gs_b).astype(F32)
    sf = e4m3_encode(np.minimum(t, FP8_MAX))
    d = (e4m3_decode(sf) * gs_b).astype(F32)
    ok = d >= FLT_MIN
    inv = np.where(ok, F32(1.0) / np.where(ok, d, F32(1.0)), F32(0.0)).astype(F32)
    v = (xb * inv[:, :, None]).astype(F32)
    nib = e2m1_encode_rne(v).reshape(M, K)
    return pack_nibbles(nib), sf, gs


def quant_mxfp4(x):
    """MXFP4: e2m1 values, one E8M0 scale per 32 K-elements.
    e = clamp(floor(log2(amax_32)) - 2, -127, 127), byte = e + 127, q = e2m1_rne(x * 2^-e).
    Returns (packed [M, K/2], scale bytes linear [M, K/32])."""
    x = _f32(x)
    M, K = x.shape
    assert K % 32 == 0
    xb = x.reshape(M, K // 32, 32)
    amax = np.max(np.abs(xb), axis=2).astype(F32)
    expf = ((amax.view(np.uint32) >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32)
    e = np.clip(expf - 127 - 2, -127, 127)
    sf = (e + 127).astype(U8)
    inv = np.ldexp(F32(1.0), -e).astype(F32)
    v = (xb * inv[:, :, None]).astype(F32)
    nib = e2m1_encode_rne(v).reshape(M, K)
    return pack_nibbles(nib), sf


# ----------------------------------------------------------------------------
# Scale-factor tile layout consumed by block-scaled tensor-core MMA
# ----------------------------------------------------------------------------

def sf_swizzled_size(rows: int, nblk: int) -> int:
    return ((rows + 127) // 128) * ((nblk + 3) // 4) * 512


def swizzle_sf(sf: np.ndarray) -> np.ndarray:
    """Linear [rows, nblk] scale bytes -> 512-byte tiles of 128 rows x 4 K-blocks.
    Tile (rt, kt) sits at (rt * ceil(nblk/4) + kt) * 512; inside a tile the byte for
    (r, c) is at (r % 32) * 16 + (r // 32) * 4 + c.  Padding bytes are zero."""
    sf = np.asarray(sf, dtype=U8)
    rows, nblk = sf.shape
    rt, kt = (rows + 127) // 128, (nblk + 3) // 4
    p = np.zeros((rt * 128, kt * 4), dtype=U8)
    p[:rows, :nblk] = sf
    # (rt, r_hi(4), r_lo(32), kt, c(4)) -> (rt, kt, r_lo, r_hi, c)
    t = p.reshape(rt, 4, 32, kt, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(-1)


def unswizzle_sf(buf: np.ndarray, rows: int, nblk: int) -> np.ndarray:
    rt, kt = (rows + 127) // 128, (nblk + 3) // 4
    t = np.asarray(buf, dtype=U8).reshape(rt, kt, 32, 4, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(rt * 128, kt * 4)[:rows, :nblk]


def swizzle_sf_grouped(sf: np.ndarray, offsets) -> np.ndarray:
    """Ragged groups: group g owns rows offsets[g]:offsets[g+1] of `sf`; each group's
    tiles start at a fresh 128-row tile (tile index = sum of ceil(M_g'/128) before it)."""
    parts = [swizzle_sf(sf[offsets[g]:offsets[g + 1]]) for g in range(len(offsets) - 1)
             if offsets[g + 1] > offsets[g]]
    return np.concatenate(parts) if parts else np.zeros(0, dtype=U8)


# ----------------------------------------------------------------------------
# Dequantise + GEMM (fp32 accumulate)
# ----------------------------------------------------------------------------

def dequant_fp4_values(packed, sf_f32_per_block, block: int) -> np.ndarray:
    """lut[q] * scale with one scale per `block` K-elements (exact in fp32 when the
    scale is an E4M3 or E8M0 value)."""
    v = e2m1_decode(unpack_nibbles(packed))
    M, K = v.shape
    return (v.reshape(M, K // block, block) * _f32(sf_f32_per_block)[:, :, None]).reshape(M, K).astype(F32)


def gemm_fp8_per_tensor(qa, qb_nk, scale_a, scale_b) -> np.ndarray:
    """(A.f32 @ B.f32) * scale_a * scale_b - tilelang/gemm/gemm_kernels.py:104-112,
    triton/gemm/gemm_kernels.py:89-97.  `qb_nk` is the K-major weight [N, K]."""
    acc = e4m3_decode(qa) @ e4m3_decode(qb_nk).T
    return ((acc * F32(scale_a)).astype(F32) * F32(scale_b)).astype(F32)


def gemm_fp8_groupwise(qa, qb_nk, sa, sb, group: int = 128) -> np.ndarray:
    """cuda/gemm/fp8_gemm.cu:84-97: per K-group partial sum, times sa[m,g]*sb[g,n], summed.
    sa [M, G]; sb [G, N] (a 128x128 block scale is sb repeated over 128 columns)."""
    A = e4m3_decode(qa)
    B = e4m3_decode(qb_nk)
    M, K = A.shape
    N = B.shape[0]
    acc = np.zeros((M, N), dtype=F32)
    for g in range((K + group - 1) // group):
        k0, k1 = g * group, min((g + 1) * group, K)
        part = A[:, k0:k1] @ B[:, k0:k1].T
        acc += ((part * _f32(sa)[:, g, None]).astype(F32) * _f32(sb)[g, None, :]).astype(F32)
    return acc


def expand_block_scale(sb_blocks: np.ndarray, N: int, block: int = 128) -> np.ndarray:
    """[ceil(N/b), ceil(K/b)] weight block scales -> [ceil(K/b), N] per-column layout."""
    return np.ascontiguousarray(np.repeat(_f32(sb_blocks), block, axis=0)[:N].T)


def gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb) -> np.ndarray:
    """Exact operands lut[q]*sf, fp32-accumulated product, times (gsa*gsb) once.  With per-token scales (gsa an array
    [M]) the product is multiplied by gsb and then, row by row, by gsa[m] - the order of the kernels' epilogue
    (global scales first, per-token factor second)."""
    A = dequant_fp4_values(pa, e4m3_decode(sfa), 16)
    B = dequant_fp4_values(pb, e4m3_decode(sfb), 16)
    if np.ndim(gsa) == 1:
        return (((A @ B.T) * F32(gsb)).astype(F32) * _f32(gsa)[:, None]).astype(F32)
    return ((A @ B.T) * F32(F32(gsa) * F32(gsb))).astype(F32)


def gemm_mxfp4(pa, sfa, pb, sfb) -> np.ndarray:
    A = dequant_fp4_values(pa, e8m0_decode(sfa), 32)
    B = dequant_fp4_values(pb, e8m0_decode(sfb), 32)
    return (A @ B.T).astype(F32)


def gemm_fp4_ref32(pa_flat, sa, pb_flat_kn, sb, M: int, N: int, K: int) -> np.ndarray:
    """cuda/gemm/fp4_gemm.cu:95-137: A packed [M,K] pairs along K, B packed [K,N] pairs
    along N, sa [M, K/32], sb [K/32, N]; C = sum_g (sum_k a*b) * sa * sb."""
    A = e2m1_decode(unpack_nibbles(np.asarray(pa_flat, dtype=U8).reshape(-1))[: M * K]).reshape(M, K)
    B = e2m1_decode(unpack_nibbles(np.asarray(pb_flat_kn, dtype=U8).reshape(-1))[: K * N]).reshape(K, N)
    acc = np.zeros((M, N), dtype=F32)
    for g in range((K + 31) // 32):
        k0, k1 = g * 32, min(g * 32 + 32, K)
        part = A[:, k0:k1] @ B[k0:k1, :]
        acc += ((part * _f32(sa).reshape(M, -1)[:, g, None]).astype(F32)
                * _f32(sb).reshape(-1, N)[g, None, :]).astype(F32)
    return acc


def bf16_round(x) -> np.ndarray:
    """fp32 -> bf16 (RNE) -> fp32."""
    b = _f32(x).view(np.uint32)
    r = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(F32)


def rel_frobenius(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / den) if den > 0 else float(np.linalg.norm(got - want))


# ---- gated activations (consumers of the gate/up projection) ---------------------------------

def silu(x) -> np.ndarray:
    """x / (1 + exp(-x)) in fp32 (cuda/activations/fused_gated_activations.cu:27-29;
    tilelang/activations/activation_kernels.py:58-59 writes it x * sigmoid(x))."""
    x = _f32(x)
    return (x / (F32(1) + np.exp(-x, dtype=F32))).astype(F32)


def gelu_tanh(x) -> np.ndarray:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (fused_gated_activations.cu:32-37), evaluated in
    fp64 and rounded once."""
    x = _f32(x).astype(np.float64)
    return (0.5 * x * (1.0 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))).astype(F32)


def swiglu(x) -> np.ndarray:
    """[B, 2H] with the gate in the first H columns -> [B, H] = silu(gate) * up
    (fused_gated_activations.cu:75-90, triton/activations/activation_kernels.py:105-115)."""
    x = _f32(x)
    h = x.shape[-1] // 2
    return (silu(x[..., :h]) * x[..., h:]).astype(F32)


def geglu(x) -> np.ndarray:
    """[B, 2H] -> [B, H] = gelu_tanh(gate) * up (fused_gated_activations.cu:92-105)."""
    x = _f32(x)
    h = x.shape[-1] // 2
    return (gelu_tanh(x[..., :h]) * x[..., h:]).astype(F32)


def interleave_gate_up(w) -> np.ndarray:
    """Weight rows [.., 2H, K] ordered [gate; up] -> gate_0, up_0, gate_1, up_1, ... (the order the fused epilogue wants)."""
    w = np.asarray(w)
    h = w.shape[-2] // 2
    return np.stack((w[..., :h, :], w[..., h:, :]), axis=-2).reshape(w.shape)


def gated_of_interleaved(full, kind: str = "swiglu") -> np.ndarray:
    """The same activations on a projection whose columns are (gate, up) pairs."""
    full = _f32(full)
    g, u = full[..., 0::2], full[..., 1::2]
    return ((silu(g) if kind == "swiglu" else gelu_tanh(g)) * u).astype(F32)
