"""ctypes front end of the split12 CPU oracle -- TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline legs may import
this module; the shipped package never does.  It wraps

* ``libsplit12_oracle.so``  -- the C restatement in ``split12_oracle.c``
* ``_ref/split12_pack_ref.so`` -- the reference's own ``split12_pack.c``
  compiled unmodified (present when the oracle was built next to an upstream
  checkout; optional everywhere else)

and adds seeded synthetic-tensor generators with the shapes and value
distributions of the benchmark configurations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsplit12_oracle.so")
_REF_PACK_PATH = os.path.join(_HERE, "_ref", "split12_pack_ref.so")


def build(force: bool = False) -> None:
    """Compile the oracle (and oracle/_ref when the upstream checkout exists)."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "split12_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, "libsplit12_oracle.so", "ref"], check=True,
                       stdout=subprocess.DEVNULL)


def _p(a, t):
    return None if a is None else a.ctypes.data_as(C.POINTER(t))


_u8, _u16, _i16, _i32, _f32 = C.c_uint8, C.c_uint16, C.c_int16, C.c_int32, C.c_float
_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.s12o_find_base_exp.restype = C.c_int
        L.s12o_find_base_exp.argtypes = [C.POINTER(_u16), C.c_int64]
        L.s12o_pack.restype = C.c_int64
        L.s12o_build_escape_table.restype = C.c_int32
        L.s12o_shard_rows.restype = C.c_int64
        L.s12o_shard_cols.restype = C.c_int64
        L.s12o_num_threads.restype = C.c_int
        _lib = L
    return _lib


def have_ref_packer() -> bool:
    return os.path.exists(_REF_PACK_PATH)


_ref = None


def ref_packer():
    """The compiled reference packer, bound exactly as engine/convert_model.py:21-38 binds it."""
    global _ref
    if _ref is None:
        R = C.CDLL(_REF_PACK_PATH)
        R.split12_find_base_exp.argtypes = [C.POINTER(_u16), C.c_int]
        R.split12_find_base_exp.restype = C.c_int
        R.pack_split12.argtypes = [C.POINTER(_u16), C.c_int, C.c_int, C.c_int,
                                   C.POINTER(_u8), C.POINTER(_u8), C.POINTER(_i32),
                                   C.POINTER(_i32), C.POINTER(_i16), C.POINTER(_i16)]
        R.pack_split12.restype = C.c_int
        _ref = R
    return _ref


@dataclass
class Packed:
    """One packed tensor on the host (the per-tensor file family of the on-disk format)."""
    M: int
    K: int
    base_exp: int
    sm: np.ndarray          # uint8 [M*K]
    gr: np.ndarray          # uint8 [M*K/2]
    row_off: np.ndarray     # int32 [M+1]
    cols: np.ndarray        # int32 [np]
    correct: np.ndarray     # int16 [np]
    wrong: np.ndarray       # int16 [np]

    @property
    def num_patches(self) -> int:
        return int(self.cols.shape[0])

    @property
    def compressed_bytes(self) -> int:
        return self.M * self.K * 3 // 2


# ----------------------------------------------------------------------------
# bf16 helpers
# ----------------------------------------------------------------------------

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << np.uint32(16)).view(np.float32)


# ----------------------------------------------------------------------------
# packer / unpack
# ----------------------------------------------------------------------------

def find_base_exp(w: np.ndarray, use_ref: bool = False) -> int:
    w = np.ascontiguousarray(w, dtype=np.uint16).ravel()
    if use_ref:
        return int(ref_packer().split12_find_base_exp(_p(w, _u16), C.c_int(w.size)))
    return int(lib().s12o_find_base_exp(_p(w, _u16), C.c_int64(w.size)))


def pack(w: np.ndarray, base_exp: int | None = None, use_ref: bool = False) -> Packed:
    """Pack bf16 bit patterns [M,K].  ``use_ref`` routes through the compiled reference packer."""
    assert w.ndim == 2 and w.dtype == np.uint16
    M, K = w.shape
    w = np.ascontiguousarray(w)
    n = M * K
    if base_exp is None:
        base_exp = find_base_exp(w, use_ref)
    sm = np.zeros(n, np.uint8)
    gr = np.zeros((n + 1) // 2, np.uint8)
    row_off = np.zeros(M + 1, np.int32)
    cap = n if n < (1 << 22) else max(n // 10, 1024)   # convert_model.py:108 uses max(n/10,1024)
    cols = np.zeros(cap, np.int32)
    correct = np.zeros(cap, np.int16)
    wrong = np.zeros(cap, np.int16)
    if use_ref:
        npat = ref_packer().pack_split12(_p(w, _u16), M, K, base_exp, _p(sm, _u8), _p(gr, _u8),
                                         _p(row_off, _i32), _p(cols, _i32), _p(correct, _i16),
                                         _p(wrong, _i16))
    else:
        npat = lib().s12o_pack(_p(w, _u16), C.c_int64(M), C.c_int64(K), C.c_int(base_exp),
                               _p(sm, _u8), _p(gr, _u8), _p(row_off, _i32), _p(cols, _i32),
                               _p(correct, _i16), _p(wrong, _i16))
    npat = int(npat)
    return Packed(M, K, int(base_exp), sm, gr, row_off, cols[:npat].copy(),
                  correct[:npat].copy(), wrong[:npat].copy())


def unpack_wrong(p: Packed) -> np.ndarray:
    out = np.empty((p.M, p.K), np.uint16)
    lib().s12o_unpack_wrong(_p(p.sm, _u8), _p(p.gr, _u8), C.c_int(p.base_exp),
                            C.c_int64(p.M), C.c_int64(p.K), _p(out, _u16))
    return out


def unpack_exact(p: Packed) -> np.ndarray:
    out = np.empty((p.M, p.K), np.uint16)
    lib().s12o_unpack_exact(_p(p.sm, _u8), _p(p.gr, _u8), C.c_int(p.base_exp),
                            _p(p.row_off, _i32), _p(p.cols, _i32), _p(p.correct, _i16),
                            C.c_int64(p.M), C.c_int64(p.K), _p(out, _u16))
    return out


def unpack_numpy(p: Packed, exact: bool = True) -> np.ndarray:
    """Independent numpy statement of the decode (second opinion on the C restatement)."""
    n = p.M * p.K
    g = np.empty(n, np.uint32)
    g[0::2] = p.gr[: n // 2] & 0xF            # even linear index -> low nibble
    g[1::2] = p.gr[: n // 2] >> 4             # odd linear index  -> high nibble
    sm = p.sm.astype(np.uint32)
    bits = ((sm >> 7) << 15) | (((np.int64(p.base_exp) + g.astype(np.int64)) << 7) & 0xFFFFFFFF).astype(np.uint32) | (sm & 0x7F)
    out = (bits & 0xFFFF).astype(np.uint16).reshape(p.M, p.K)
    if exact and p.num_patches:
        rows = np.repeat(np.arange(p.M), np.diff(p.row_off))
        out[rows, p.cols] = p.correct.view(np.uint16)
    return out


# ----------------------------------------------------------------------------
# escape table (batch4/8 path) and sharding
# ----------------------------------------------------------------------------

def build_escape_table(p: Packed, with_counts: bool = True):
    row_base = np.zeros(p.M, np.int32)
    counts = np.zeros(p.M * 256, np.uint8) if with_counts else None
    vals = np.zeros(max(p.num_patches, 1), np.int16)
    nonempty = np.zeros(p.M, np.int32)
    nne = lib().s12o_build_escape_table(_p(p.row_off, _i32), _p(p.cols, _i32), _p(p.correct, _i16),
                                        C.c_int64(p.M), _p(row_base, _i32), _p(counts, _u8),
                                        _p(vals, _i16), _p(nonempty, _i32))
    return row_base, counts, vals[: p.num_patches], nonempty[:nne].copy()


def shard_rows(p: Packed, r0: int, r1: int) -> Packed:
    Ms = r1 - r0
    sm = np.empty(Ms * p.K, np.uint8); gr = np.empty(Ms * p.K // 2, np.uint8)
    ro = np.empty(Ms + 1, np.int32)
    cap = max(p.num_patches, 1)
    co = np.empty(cap, np.int32); cv = np.empty(cap, np.int16); wv = np.empty(cap, np.int16)
    n = lib().s12o_shard_rows(_p(p.sm, _u8), _p(p.gr, _u8), _p(p.row_off, _i32), _p(p.cols, _i32),
                              _p(p.correct, _i16), _p(p.wrong, _i16), C.c_int64(p.K),
                              C.c_int64(r0), C.c_int64(r1), _p(sm, _u8), _p(gr, _u8), _p(ro, _i32),
                              _p(co, _i32), _p(cv, _i16), _p(wv, _i16))
    return Packed(Ms, p.K, p.base_exp, sm, gr, ro, co[:n].copy(), cv[:n].copy(), wv[:n].copy())


def shard_cols(p: Packed, c0: int, c1: int) -> Packed:
    Ks = c1 - c0
    sm = np.empty(p.M * Ks, np.uint8); gr = np.empty(p.M * Ks // 2, np.uint8)
    ro = np.empty(p.M + 1, np.int32)
    cap = max(p.num_patches, 1)
    co = np.empty(cap, np.int32); cv = np.empty(cap, np.int16); wv = np.empty(cap, np.int16)
    n = lib().s12o_shard_cols(_p(p.sm, _u8), _p(p.gr, _u8), _p(p.row_off, _i32), _p(p.cols, _i32),
                              _p(p.correct, _i16), _p(p.wrong, _i16), C.c_int64(p.M), C.c_int64(p.K),
                              C.c_int64(c0), C.c_int64(c1), _p(sm, _u8), _p(gr, _u8), _p(ro, _i32),
                              _p(co, _i32), _p(cv, _i16), _p(wv, _i16))
    return Packed(p.M, Ks, p.base_exp, sm, gr, ro, co[:n].copy(), cv[:n].copy(), wv[:n].copy())


# ----------------------------------------------------------------------------
# GEMV / GEMM checkers and the timed CPU baseline
# ----------------------------------------------------------------------------

def gemm_twopass(p: Packed, X: np.ndarray, patches: bool = True) -> np.ndarray:
    """fp32 [B,M]: first pass with wrong escapes, then the (correct-wrong)*x correction."""
    X = np.ascontiguousarray(X, np.uint16)
    B, K = X.shape
    assert K == p.K
    out = np.empty((B, p.M), np.float32)
    use = patches and p.num_patches > 0
    lib().s12o_gemm_twopass(_p(p.sm, _u8), _p(p.gr, _u8), C.c_int(p.base_exp),
                            _p(p.row_off, _i32) if use else None,
                            _p(p.cols, _i32) if use else None,
                            _p(p.correct, _i16) if use else None,
                            _p(p.wrong, _i16) if use else None,
                            _p(X, _u16), C.c_int64(K), _p(out, _f32), C.c_int64(p.M),
                            C.c_int64(p.M), C.c_int64(p.K), C.c_int64(B))
    return out


def gemm_exact(W: np.ndarray, X: np.ndarray) -> np.ndarray:
    W = np.ascontiguousarray(W, np.uint16); X = np.ascontiguousarray(X, np.uint16)
    M, K = W.shape; B = X.shape[0]
    out = np.empty((B, M), np.float32)
    lib().s12o_gemm_exact(_p(W, _u16), _p(X, _u16), C.c_int64(K), _p(out, _f32), C.c_int64(M),
                          C.c_int64(M), C.c_int64(K), C.c_int64(B))
    return out


def gemm_abs(W: np.ndarray, X: np.ndarray) -> np.ndarray:
    W = np.ascontiguousarray(W, np.uint16); X = np.ascontiguousarray(X, np.uint16)
    M, K = W.shape; B = X.shape[0]
    out = np.empty((B, M), np.float32)
    lib().s12o_gemm_abs(_p(W, _u16), _p(X, _u16), C.c_int64(K), _p(out, _f32), C.c_int64(M),
                        C.c_int64(M), C.c_int64(K), C.c_int64(B))
    return out


def cpu_unpack_gemm_f32(p: Packed, X: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
    """The timed CPU baseline: lossless unpack + fp32 GEMM on all host threads."""
    X = np.ascontiguousarray(X, np.uint16)
    B, K = X.shape
    if out is None:
        out = np.empty((B, p.M), np.float32)
    use = p.num_patches > 0
    lib().s12o_cpu_unpack_gemm_f32(_p(p.sm, _u8), _p(p.gr, _u8), C.c_int(p.base_exp),
                                   _p(p.row_off, _i32) if use else None,
                                   _p(p.cols, _i32) if use else None,
                                   _p(p.correct, _i16) if use else None,
                                   _p(X, _u16), C.c_int64(K), _p(out, _f32), C.c_int64(p.M),
                                   C.c_int64(p.M), C.c_int64(p.K), C.c_int64(B))
    return out


def num_threads() -> int:
    return int(lib().s12o_num_threads())


def set_num_threads(n: int) -> int:
    """Team size of the oracle's parallel loops, whatever OMP_NUM_THREADS says; returns the size in effect."""
    L = lib()
    L.s12o_set_num_threads.restype = C.c_int
    return int(L.s12o_set_num_threads(C.c_int(int(n))))


# ----------------------------------------------------------------------------
# seeded synthetic tensors (stand-ins for real checkpoints)
# ----------------------------------------------------------------------------

def synth_weights(M: int, K: int, seed: int, std: float = 0.02,
                  outlier_frac: float = 0.0, outlier_scale: float = 100.0) -> np.ndarray:
    """bf16 bit patterns of N(0,std) weights with a Bernoulli(outlier_frac) mask scaled up."""
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((M, K), dtype=np.float32) * np.float32(std)
    if outlier_frac > 0:
        mask = rng.random((M, K), dtype=np.float32) < outlier_frac
        w = np.where(mask, w * np.float32(outlier_scale), w)
    return f32_to_bf16_bits(w)


def synth_acts(B: int, K: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed + 7919)
    return f32_to_bf16_bits(rng.standard_normal((B, K), dtype=np.float32))
