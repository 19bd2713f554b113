"""Host-side mirror of the Turbo-Lossless engine's interface to the split12 kernels.

``CompressedWeight`` has the fields of the engine's struct of the same name
(engine/model.h:21-40 of the reference) and is loaded from the same per-tensor
file family (engine/model.cpp:32-163).  ``Split12Engine`` offers one method per
call-site macro of engine/inference.cpp (MATVEC_B1_NOPATCH, NV_OR_HIP_PATCHES,
BATCH4/8_MATVEC, GEMM_ONLY, PATCHES_ASYNC) plus the fused superset calls, each a
thin wrapper over one C-ABI entry point.  torch is used for device memory and
streams only.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import capi
from .capi import S12PatchBatchDesc, S12Tensor, check


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(stream=None) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream if isinstance(stream, int) else stream.cuda_stream


@dataclass
class CompressedWeight:
    """One packed tensor resident on a device (engine/model.h:21-40)."""
    M: int
    K: int
    base_exp: int
    split_sm: torch.Tensor                     # uint8 [M*K]
    split_gr: torch.Tensor                     # uint8 [M*K/2]
    num_patches: int = 0
    row_offsets: Optional[torch.Tensor] = None     # int32 [M+1]
    patch_cols: Optional[torch.Tensor] = None      # int32 [np]
    patch_correct: Optional[torch.Tensor] = None   # int16 [np]
    patch_wrong: Optional[torch.Tensor] = None     # int16 [np]
    escape_row_base: Optional[torch.Tensor] = None  # int32 [M]
    escape_counts: Optional[torch.Tensor] = None    # uint8 [M*256], only when asked for
    escape_vals: Optional[torch.Tensor] = None      # int16 [np], (row, col%256, col) order
    patch_nonempty_rows: Optional[torch.Tensor] = None  # int32 [num_nonempty_rows]
    num_nonempty_rows: int = 0
    _keep: list = field(default_factory=list, repr=False)

    # -- construction ------------------------------------------------------
    @classmethod
    def from_host(cls, M: int, K: int, base_exp: int, sm: np.ndarray, gr: np.ndarray,
                  row_off: Optional[np.ndarray], cols: Optional[np.ndarray],
                  correct: Optional[np.ndarray], wrong: Optional[np.ndarray],
                  device="cuda", escape_table: bool = True, escape_counts: bool = False) -> "CompressedWeight":
        """Uploads one packed tensor; builds the escape table and non-empty row list on the host
        (the load-time steps of engine/model.cpp:86-156) with the library's host helper."""
        dev = torch.device(device)
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
        npat = 0 if cols is None else int(cols.shape[0])
        w = cls(M=M, K=K, base_exp=int(base_exp), split_sm=up(sm), split_gr=up(gr), num_patches=npat)
        if npat > 0 and row_off is not None:
            w.row_offsets, w.patch_cols = up(row_off), up(cols)
            w.patch_correct, w.patch_wrong = up(correct), up(wrong)
            if escape_table:
                lib = capi.load()
                row_base = np.zeros(M, np.int32)
                counts = np.zeros(M * 256, np.uint8) if escape_counts else None
                vals = np.zeros(npat, np.int16)
                nonempty = np.zeros(M, np.int32)
                ro = np.ascontiguousarray(row_off, np.int32)
                co = np.ascontiguousarray(cols, np.int32)
                cv = np.ascontiguousarray(correct, np.int16)
                nne = lib.s12_host_build_escape_table(
                    ro.ctypes.data, co.ctypes.data, cv.ctypes.data, M, row_base.ctypes.data,
                    None if counts is None else counts.ctypes.data, vals.ctypes.data, nonempty.ctypes.data)
                if nne < 0:
                    raise capi.S12Error(f"s12_host_build_escape_table failed with {nne}")
                w.escape_row_base, w.escape_vals = up(row_base), up(vals)
                if counts is not None:
                    w.escape_counts = up(counts)
                w.num_nonempty_rows = int(nne)
                if nne > 0:
                    w.patch_nonempty_rows = up(nonempty[:nne])
        return w

    @classmethod
    def from_packed(cls, p, device="cuda", **kw) -> "CompressedWeight":
        """From any object with fields M, K, base_exp, sm, gr, row_off, cols, correct, wrong."""
        return cls.from_host(p.M, p.K, p.base_exp, p.sm, p.gr, p.row_off, p.cols, p.correct, p.wrong,
                             device=device, **kw)

    @classmethod
    def from_dir(cls, directory: str, prefix: str, device="cuda", **kw) -> "CompressedWeight":
        """Reads ``<prefix>.dims`` (text ``M K num_patches base_exp``) and the six binary files
        written by engine/convert_model.py:127-134; missing or empty CSR files mean no escapes."""
        with open(os.path.join(directory, prefix + ".dims")) as f:
            parts = f.read().split()
        if len(parts) < 3:
            raise ValueError(f"{prefix}.dims: expected 'M K num_patches [base_exp]'")
        M, K, npat = int(parts[0]), int(parts[1]), int(parts[2])
        base_exp = int(parts[3]) if len(parts) > 3 else 0

        def rd(suffix, dtype):
            path = os.path.join(directory, f"{prefix}.{suffix}.bin")
            if not os.path.exists(path) or os.path.getsize(path) == 0:
                return None
            return np.fromfile(path, dtype=dtype)

        sm, gr = rd("sm", np.uint8), rd("gr", np.uint8)
        if sm is None or gr is None:
            raise FileNotFoundError(f"split12 files missing for {prefix} (need .sm.bin + .gr.bin)")
        if sm.size != M * K or gr.size != (M * K + 1) // 2:
            raise ValueError(f"{prefix}: sm/gr sizes do not match dims {M}x{K}")
        ro, co = rd("row_off", np.int32), rd("patch_cols", np.int32)
        cv, wv = rd("patch_correct", np.int16), rd("patch_wrong", np.int16)
        if npat > 0 and (ro is None or co is None or cv is None or wv is None):
            raise ValueError(f"{prefix}: {npat} escapes declared but CSR files are missing")
        if npat > 0 and (ro.size != M + 1 or co.size != npat or cv.size != npat or wv.size != npat):
            raise ValueError(f"{prefix}: CSR file sizes do not match dims")
        if npat == 0:
            ro = co = cv = wv = None
        return cls.from_host(M, K, base_exp, sm, gr, ro, co, cv, wv, device=device, **kw)

    @classmethod
    def pack_on_device(cls, w_bf16: torch.Tensor, base_exp: Optional[int] = None,
                       escape_table: bool = False) -> "CompressedWeight":
        """Packs a bf16 [M,K] tensor that already lives on the device with the library's packer
        kernels (same bytes as split12_find_base_exp + pack_split12 of the reference)."""
        assert w_bf16.is_cuda and w_bf16.dim() == 2 and w_bf16.dtype in (torch.bfloat16, torch.int16)
        lib = capi.load()
        w = w_bf16.contiguous()
        M, K = w.shape
        dev = w.device
        st = _stream()
        if base_exp is None:
            hist = torch.empty(256, dtype=torch.int64, device=dev)
            check(lib.s12_pack_histogram_async(w.data_ptr(), M * K, hist.data_ptr(), st), "s12_pack_histogram_async")
            h = np.ascontiguousarray(hist.cpu().numpy().astype(np.uint64))
            base_exp = int(lib.s12_pack_find_base_exp_host(h.ctypes.data))
        sm = torch.empty(M * K, dtype=torch.uint8, device=dev)
        gr = torch.empty(M * K // 2, dtype=torch.uint8, device=dev)
        row_off = torch.empty(M + 1, dtype=torch.int32, device=dev)
        check(lib.s12_pack_async(w.data_ptr(), M, K, base_exp, sm.data_ptr(), gr.data_ptr(), row_off.data_ptr(), st),
              "s12_pack_async")
        npat = int(row_off[-1].item())
        out = cls(M=M, K=K, base_exp=base_exp, split_sm=sm, split_gr=gr, num_patches=npat)
        if npat > 0:
            cols = torch.empty(npat, dtype=torch.int32, device=dev)
            correct = torch.empty(npat, dtype=torch.int16, device=dev)
            wrong = torch.empty(npat, dtype=torch.int16, device=dev)
            check(lib.s12_pack_fill_async(w.data_ptr(), M, K, base_exp, row_off.data_ptr(), cols.data_ptr(),
                                          correct.data_ptr(), wrong.data_ptr(), st), "s12_pack_fill_async")
            out.row_offsets, out.patch_cols, out.patch_correct, out.patch_wrong = row_off, cols, correct, wrong
            if escape_table:
                out.build_escape_table_on_device()
        return out

    def build_escape_table_on_device(self, escape_counts: bool = False, stream=None) -> None:
        """Escape table of the batch4/8 path and the non-empty row list, built by kernels from the CSR list that
        is already on the device (the load-time passes of engine/model.cpp:86-156 without the host)."""
        if self.num_patches <= 0 or self.row_offsets is None:
            return
        lib = capi.load()
        dev = self.split_sm.device
        self.escape_row_base = torch.empty(self.M, dtype=torch.int32, device=dev)
        self.escape_vals = torch.empty(self.num_patches, dtype=torch.int16, device=dev)
        self.escape_counts = torch.empty(self.M * 256, dtype=torch.uint8, device=dev) if escape_counts else None
        rows = torch.empty(self.M, dtype=torch.int32, device=dev)
        count = torch.zeros(1, dtype=torch.int32, device=dev)
        check(lib.s12_build_escape_table_async(
            self.row_offsets.data_ptr(), self.patch_cols.data_ptr(), self.patch_correct.data_ptr(), self.M,
            self.escape_row_base.data_ptr(), _ptr(self.escape_counts), self.escape_vals.data_ptr(),
            rows.data_ptr(), count.data_ptr(), _stream(stream)), "s12_build_escape_table_async")
        self.num_nonempty_rows = int(count.item())
        self.patch_nonempty_rows = rows[: self.num_nonempty_rows] if self.num_nonempty_rows else None

    @classmethod
    def load(cls, directory: str, prefix: str, device="cuda", escape_table: bool = True, escape_counts: bool = False,
             stream=None) -> "CompressedWeight":
        """Loads ``<prefix>.*`` of a converted model directory with the library's native loader
        (``s12_load_tensor``: pinned double-buffered uploads, escape table and row list built on the device).
        Same file family and error behaviour as ``load_compressed`` of engine/model.cpp:32-163."""
        lib = capi.load()
        M, K, be, npat = C.c_int(), C.c_int(), C.c_int(), C.c_int64()
        d, pfx = os.fsencode(directory), prefix.encode()
        check(lib.s12_tensor_dims(d, pfx, C.byref(M), C.byref(K), C.byref(npat), C.byref(be)), "s12_tensor_dims")
        M, K, be, npat = M.value, K.value, be.value, npat.value
        dev = torch.device(device)
        e = lambda n, dt: torch.empty(n, dtype=dt, device=dev)  # noqa: E731
        w = cls(M=M, K=K, base_exp=be, split_sm=e(M * K, torch.uint8), split_gr=e((M * K + 1) // 2, torch.uint8))
        ro = co = cv = wv = rb = ec = ev = ne = None
        if npat > 0:
            ro, co, cv, wv = e(M + 1, torch.int32), e(npat, torch.int32), e(npat, torch.int16), e(npat, torch.int16)
            if escape_table:
                rb, ev, ne = e(M, torch.int32), e(npat, torch.int16), e(M, torch.int32)
                ec = e(M * 256, torch.uint8) if escape_counts else None
        nne = C.c_int(0)
        with torch.cuda.device(dev):
            got = lib.s12_load_tensor(d, pfx, w.split_sm.data_ptr(), w.split_gr.data_ptr(), _ptr(ro), _ptr(co), _ptr(cv),
                                      _ptr(wv), _ptr(rb), _ptr(ec), _ptr(ev), _ptr(ne), C.byref(nne), _stream(stream))
        if got < 0:
            check(int(got), "s12_load_tensor")
        if got > 0:
            w.num_patches = int(got)
            w.row_offsets, w.patch_cols, w.patch_correct, w.patch_wrong = ro, co, cv, wv
            if escape_table:
                w.escape_row_base, w.escape_counts, w.escape_vals = rb, ec, ev
                w.num_nonempty_rows = nne.value
                w.patch_nonempty_rows = ne[: nne.value] if nne.value else None
        return w

    # -- views -----------------------------------------------------------------
    def tensor(self, with_csr: bool = True) -> S12Tensor:
        t = S12Tensor()
        t.sm, t.gr = self.split_sm.data_ptr(), self.split_gr.data_ptr()
        t.M, t.K, t.base_exp, t.num_patches = self.M, self.K, self.base_exp, self.num_patches
        if with_csr and self.num_patches > 0 and self.row_offsets is not None:
            t.row_off, t.cols = self.row_offsets.data_ptr(), self.patch_cols.data_ptr()
            t.correct, t.wrong = self.patch_correct.data_ptr(), self.patch_wrong.data_ptr()
        else:
            t.num_patches = 0 if not with_csr else self.num_patches
        return t

    @property
    def compressed_bytes(self) -> int:
        return self.M * self.K * 3 // 2


class Split12Engine:
    """Call sites of the engine, one method per macro of engine/inference.cpp."""

    def __init__(self):
        self.lib = capi.load()

    # ---- B = 1, legacy two-pass (engine/inference.cpp:222-243) ------------------
    def matvec_b1_nopatch(self, w: CompressedWeight, bf16_in: torch.Tensor, fp32_out: torch.Tensor,
                          stream=None, portable: bool = False) -> None:
        fn = self.lib.launch_split12_v2_async if portable else self.lib.nv_launch_split12_v2_async
        check(fn(_ptr(w.split_sm), _ptr(w.split_gr), w.base_exp, _ptr(bf16_in), _ptr(fp32_out),
                 w.M, w.K, _stream(stream)), "split12_v2_async")

    def patches(self, w: CompressedWeight, bf16_in: torch.Tensor, fp32_out: torch.Tensor,
                stream=None, portable: bool = False) -> None:
        if w.num_patches <= 0 or w.row_offsets is None:
            return
        fn = self.lib.launch_patches_v2_async if portable else self.lib.nv_launch_patches_async
        check(fn(_ptr(w.row_offsets), _ptr(w.patch_cols), _ptr(w.patch_correct), _ptr(w.patch_wrong),
                 _ptr(bf16_in), _ptr(fp32_out), w.M, _stream(stream)), "patches_async")

    def matvec_dual(self, wa: CompressedWeight, wb: CompressedWeight, bf16_in: torch.Tensor,
                    out_a: torch.Tensor, out_b: torch.Tensor, stream=None, portable: bool = False) -> None:
        fn = self.lib.launch_split12_v2_dual_async if portable else self.lib.nv_launch_split12_v2_dual_async
        check(fn(_ptr(wa.split_sm), _ptr(wa.split_gr), wa.base_exp, _ptr(wb.split_sm), _ptr(wb.split_gr),
                 wb.base_exp, _ptr(bf16_in), _ptr(out_a), _ptr(out_b), wa.M, wa.K, _stream(stream)),
              "split12_v2_dual_async")

    def patches_b1_batched(self, items: Sequence[tuple], stream=None) -> None:
        """items: (weight, bf16_in, fp32_out) triples, at most 8 (fill_patch_desc, inference.cpp:54-66)."""
        descs = (S12PatchBatchDesc * 8)()
        n, max_m = 0, 0
        for w, x, o in items:
            if w.num_patches <= 0 or w.row_offsets is None:
                continue
            d = descs[n]
            d.row_offsets, d.patch_cols = _ptr(w.row_offsets), _ptr(w.patch_cols)
            d.patch_correct, d.patch_wrong = _ptr(w.patch_correct), _ptr(w.patch_wrong)
            d.activations, d.output, d.M = _ptr(x), _ptr(o), w.M
            max_m = max(max_m, w.M)
            n += 1
        check(self.lib.launch_patches_b1_batched_async(None, C.addressof(descs), n, max_m, _stream(stream)),
              "launch_patches_b1_batched_async")

    # ---- B = 4 / 8 with the escape table (engine/inference.cpp:72-81,369-382) ------
    def batch_matvec(self, w: CompressedWeight, ins: Sequence[torch.Tensor], outs: Sequence[torch.Tensor],
                     stream=None) -> None:
        n = len(ins)
        if n not in (4, 8) or len(outs) != n:
            raise ValueError("batch_matvec takes 4 or 8 activation/output vectors")
        fn = self.lib.launch_split12_batch4_async if n == 4 else self.lib.launch_split12_batch8_async
        check(fn(_ptr(w.split_sm), _ptr(w.split_gr), w.base_exp, *[_ptr(t) for t in ins],
                 _ptr(w.escape_row_base), _ptr(w.escape_counts), _ptr(w.escape_vals),
                 *[_ptr(t) for t in outs], w.M, w.K, _stream(stream)), f"launch_split12_batch{n}_async")

    # ---- batched, legacy two-pass (engine/inference.cpp:540-570) -----------------
    def gemm_only(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, n_in: int,
                  n_out: int, bs: int, stream=None, v3: bool = False, patched: bool = False) -> None:
        fn = self.lib.nv_launch_split12_fused_gemm_v3_async if v3 else self.lib.nv_launch_split12_fused_gemm_async
        pp = [None] * 4
        if patched and w.num_patches > 0:
            pp = [_ptr(w.row_offsets), _ptr(w.patch_cols), _ptr(w.patch_correct), _ptr(w.patch_wrong)]
        check(fn(_ptr(w.split_sm), _ptr(w.split_gr), w.base_exp, _ptr(bf16_in), n_in, _ptr(out), n_out,
                 w.M, w.K, bs, _stream(stream), *pp), "nv_launch_split12_fused_gemm_async")

    def gemm_cublas_path(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, n_in: int,
                         n_out: int, bs: int, weight_buf: Optional[torch.Tensor] = None,
                         weight_buf_half: int = 0, stream=None) -> None:
        check(self.lib.nv_launch_split12_cublas_batch_async(
            _ptr(w.split_sm), _ptr(w.split_gr), w.base_exp, _ptr(bf16_in), n_in, _ptr(out), n_out,
            _ptr(weight_buf), weight_buf_half, w.M, w.K, bs, _stream(stream)),
            "nv_launch_split12_cublas_batch_async")

    def patches_batch(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, n_in: int,
                      n_out: int, bs: int, stream=None) -> None:
        if w.num_nonempty_rows <= 0:
            return
        check(self.lib.nv_launch_patches_batch_async(
            _ptr(w.row_offsets), _ptr(w.patch_cols), _ptr(w.patch_correct), _ptr(w.patch_wrong),
            _ptr(w.patch_nonempty_rows), w.num_nonempty_rows, _ptr(bf16_in), n_in, _ptr(out), n_out,
            bs, _stream(stream)), "nv_launch_patches_batch_async")

    # ---- fused superset --------------------------------------------------------------
    def gemv(self, ws: Sequence[CompressedWeight], bf16_in: torch.Tensor, outs: Sequence[torch.Tensor],
             stream=None, exact: bool = True) -> None:
        """Up to four tensors sharing one activation vector, escapes corrected in the same launch."""
        n = len(ws)
        arr = (S12Tensor * n)(*[w.tensor(with_csr=exact) for w in ws])
        optr = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        check(self.lib.s12_gemv_async(arr, n, _ptr(bf16_in), optr, _stream(stream)), "s12_gemv_async")

    def gemv_batched(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, act_stride: int,
                     out_stride: int, bs: int, stream=None, exact: bool = True) -> None:
        t = w.tensor(with_csr=exact)
        check(self.lib.s12_gemv_batched_async(C.byref(t), _ptr(bf16_in), act_stride, _ptr(out), out_stride,
                                              bs, _stream(stream)), "s12_gemv_batched_async")

    def gemm(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, act_stride: int,
             out_stride: int, bs: int, stream=None, exact: bool = True) -> None:
        t = w.tensor(with_csr=exact)
        check(self.lib.s12_gemm_async(C.byref(t), _ptr(bf16_in), act_stride, _ptr(out), out_stride, bs,
                                      _stream(stream)), "s12_gemm_async")

    def gemm_multi(self, ws: Sequence[CompressedWeight], bf16_in: torch.Tensor, outs: Sequence[torch.Tensor],
                   act_stride: int, bs: int, stream=None, exact: bool = True) -> None:
        """Up to four tensors sharing the activations (q/k/v, gate/up) as one tensor-core launch."""
        n = len(ws)
        arr = (S12Tensor * n)(*[w.tensor(with_csr=exact) for w in ws])
        optr = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        strides = (C.c_int * n)(*[o.stride(0) for o in outs])
        check(self.lib.s12_gemm_multi_async(arr, n, _ptr(bf16_in), act_stride, optr, strides, bs, _stream(stream)),
              "s12_gemm_multi_async")

    def gemm_grouped(self, ws: Sequence[CompressedWeight], bf16_in: torch.Tensor, act_row0: Sequence[int],
                     outs: Sequence[torch.Tensor], act_stride: int, bs: int, stream=None, exact: bool = True) -> None:
        """Tensors that share K, each reading its own block of ``bs`` rows of ``bf16_in`` starting at
        ``act_row0[i]`` (the experts of an MoE layer): eight tensors per tensor-core launch."""
        n = len(ws)
        arr = (S12Tensor * n)(*[w.tensor(with_csr=exact) for w in ws])
        optr = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        strides = (C.c_int * n)(*[o.stride(0) for o in outs])
        rows = (C.c_int * n)(*[int(r) for r in act_row0])
        check(self.lib.s12_gemm_grouped_async(arr, n, _ptr(bf16_in), act_stride, rows, optr, strides, bs, _stream(stream)),
              "s12_gemm_grouped_async")

    def gemm_noalloc(self, w: CompressedWeight, bf16_in: torch.Tensor, out: torch.Tensor, act_stride: int,
                     out_stride: int, bs: int, stream=None, exact: bool = True) -> None:
        """s12_gemm_async for callers that may not allocate: scratch is a fixed array in the library."""
        t = w.tensor(with_csr=exact)
        check(self.lib.s12_gemm_noalloc_async(C.byref(t), _ptr(bf16_in), act_stride, _ptr(out), out_stride, bs,
                                              _stream(stream)), "s12_gemm_noalloc_async")

    def decompress(self, w: CompressedWeight, out: Optional[torch.Tensor] = None, stream=None,
                   exact: bool = True) -> torch.Tensor:
        """Lossless bf16 [M,K] (int16 storage); with exact=False escapes keep the "wrong" value."""
        if out is None:
            out = torch.empty((w.M, w.K), dtype=torch.int16, device=w.split_sm.device)
        t = w.tensor(with_csr=exact)
        check(self.lib.s12_decompress_async(C.byref(t), _ptr(out), _stream(stream)), "s12_decompress_async")
        return out

    # ---- the decode step around the projections (engine/kernels.hip launchers, same argument order) ----
    def embed_lookup(self, table_bf16: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        n_vocab, n_embd = table_bf16.shape
        check(self.lib.launch_embed_lookup(_ptr(table_bf16), _ptr(token_ids), _ptr(out), n_embd, token_ids.numel(),
                                           n_vocab, _stream(stream)), "launch_embed_lookup")

    def argmax(self, logits: torch.Tensor, result: torch.Tensor, stream=None) -> None:
        batch, n = (1, logits.numel()) if logits.dim() == 1 else logits.shape
        check(self.lib.launch_argmax_batch(_ptr(logits), _ptr(result), n, batch, _stream(stream)), "launch_argmax_batch")

    def rms_norm_bf16(self, x: torch.Tensor, weight: torch.Tensor, y_bf16: torch.Tensor, eps: float, batch: int = 1,
                      residual: Optional[torch.Tensor] = None, stream=None) -> None:
        n = weight.numel()
        if residual is None:
            check(self.lib.launch_rms_norm_bf16_batch(_ptr(x), _ptr(weight), _ptr(y_bf16), n, eps, batch, _stream(stream)),
                  "launch_rms_norm_bf16_batch")
        else:                                  # x += residual in place, then the norm of the sum
            check(self.lib.launch_add_rms_norm_bf16_batch(_ptr(x), _ptr(residual), _ptr(weight), _ptr(y_bf16), n, eps,
                                                          batch, _stream(stream)), "launch_add_rms_norm_bf16_batch")

    def silu_mul_bf16(self, gate: torch.Tensor, up: torch.Tensor, out_bf16: torch.Tensor, n: int, batch: int = 1,
                      stream=None) -> None:
        check(self.lib.launch_silu_mul_bf16_batch(_ptr(gate), _ptr(up), _ptr(out_bf16), n, batch, _stream(stream)),
              "launch_silu_mul_bf16_batch")

    def add(self, y: torch.Tensor, x: torch.Tensor, n: int, batch: int = 1, stream=None) -> None:
        check(self.lib.launch_add_batch(_ptr(y), _ptr(x), n, batch, _stream(stream)), "launch_add_batch")

    def rope_store_kv(self, q, k, v, kv_k, kv_v, scale_k, scale_v, head_dim: int, n_head: int, n_head_kv: int,
                      position: int, max_seq: int, theta: float, stream=None) -> None:
        check(self.lib.launch_rope_store_kv(_ptr(q), _ptr(k), _ptr(v), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                            head_dim, n_head, n_head_kv, position, max_seq, theta, _stream(stream)),
              "launch_rope_store_kv")

    def rope_batch(self, q, k, positions, head_dim: int, n_head: int, n_head_kv: int, theta: float, batch: int,
                   stream=None) -> None:
        check(self.lib.launch_rope_batch(_ptr(q), _ptr(k), _ptr(positions), head_dim, n_head, n_head_kv, n_head * head_dim,
                                         n_head_kv * head_dim, theta, batch, _stream(stream)), "launch_rope_batch")

    def store_kv_batch(self, k, v, kv_k, kv_v, scale_k, scale_v, positions, n_head_kv: int, head_dim: int, batch: int,
                       kv_stride: int = 0, max_seq: int = 0, stream=None) -> None:
        if kv_stride == 0:
            check(self.lib.launch_store_kv_batch(_ptr(k), _ptr(v), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                                 _ptr(positions), n_head_kv * head_dim, max_seq, n_head_kv, head_dim, batch,
                                                 _stream(stream)), "launch_store_kv_batch")
        else:
            check(self.lib.s12_store_kv_batch(_ptr(k), _ptr(v), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                              _ptr(positions), n_head_kv, head_dim, kv_stride, batch, _stream(stream)),
                  "s12_store_kv_batch")

    def rope_store_kv_batch(self, q, k, v, kv_k, kv_v, scale_k, scale_v, positions, head_dim: int, n_head: int,
                            n_head_kv: int, kv_stride: int, theta: float, batch: int, stream=None) -> None:
        check(self.lib.s12_rope_store_kv_batch(_ptr(q), _ptr(k), _ptr(v), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                               _ptr(positions), head_dim, n_head, n_head_kv, kv_stride, theta, batch,
                                               _stream(stream)), "s12_rope_store_kv_batch")

    def attention_all_heads(self, q, kv_k, kv_v, scale_k, scale_v, out_bf16, n_head: int, n_head_kv: int, head_dim: int,
                            seq_len: int, max_seq: int, scale: float, stream=None) -> None:
        check(self.lib.launch_attention_all_heads(_ptr(q), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                                  _ptr(out_bf16), n_head, n_head_kv, head_dim, seq_len, max_seq, scale,
                                                  _stream(stream)), "launch_attention_all_heads")

    def attention_all_heads_batch(self, q, kv_k, kv_v, scale_k, scale_v, out_bf16, positions, n_head: int, n_head_kv: int,
                                  head_dim: int, max_len: int, scale: float, batch: int, kv_stride: int, stream=None) -> None:
        check(self.lib.launch_attention_all_heads_batch(_ptr(q), _ptr(kv_k), _ptr(kv_v), _ptr(scale_k), _ptr(scale_v),
                                                        _ptr(out_bf16), _ptr(positions), n_head, n_head_kv, head_dim, max_len,
                                                        scale, batch, kv_stride, _stream(stream)),
              "launch_attention_all_heads_batch")

    def init(self) -> None:
        """Per-device set-up ahead of the first call (s12_init): status word, GEMM workspace, kernel attributes."""
        check(self.lib.s12_init(), "s12_init")

    def set_dependent_launch(self, enable: bool) -> bool:
        return bool(self.lib.s12_set_dependent_launch(1 if enable else 0))

    def device_status(self) -> int:
        return int(self.lib.s12_device_status())


class TPComm:
    """All-reduce of fp32 partial results across tensor-parallel ranks (s12_comm_* of the C ABI).

    One process per GPU: ``TPComm(rank, world, max_floats, group)`` allocates this rank's receive
    area, exchanges the handles with an ``all_gather_object`` on the given ``torch.distributed``
    group (the plumbing), and maps the peers' areas; ``all_reduce`` is then one kernel of this
    library on the caller's stream.  ``TPComm.local(world, max_floats)`` builds ``world``
    communicators inside one process on one device for tests.
    """

    def __init__(self, rank: int, world: int, max_floats: int, group=None, _connect: bool = True):
        self.lib = capi.load()
        self.rank, self.world, self.max_floats = rank, world, max_floats
        self._h = C.c_void_p()
        nbytes = int(self.lib.s12_comm_handle_bytes())
        handle = C.create_string_buffer(nbytes)
        check(self.lib.s12_comm_create(rank, world, max_floats, C.byref(self._h), handle), "s12_comm_create")
        if _connect:
            if world > 1:
                import torch.distributed as dist
                gathered = [None] * world
                dist.all_gather_object(gathered, handle.raw, group=group)
                blob = b"".join(gathered)
            else:
                blob = handle.raw
            check(self.lib.s12_comm_connect(self._h, blob), "s12_comm_connect")

    @classmethod
    def local(cls, world: int, max_floats: int):
        comms = [cls(r, world, max_floats, _connect=False) for r in range(world)]
        arr = (C.c_void_p * world)(*[c._h for c in comms])
        check(comms[0].lib.s12_comm_connect_local(arr, world), "s12_comm_connect_local")
        return comms

    def all_reduce(self, src: torch.Tensor, dst: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        dst = src if dst is None else dst
        check(self.lib.s12_allreduce_f32_async(self._h, _ptr(src), _ptr(dst), src.numel(), _stream(stream)),
              "s12_allreduce_f32_async")
        return dst

    def gemv_all_reduce(self, w: "CompressedWeight", bf16_in: torch.Tensor, out: torch.Tensor, stream=None,
                        exact: bool = True) -> None:
        """Row-parallel shard x activations and the sum over ranks as one kernel (B = 1)."""
        t = w.tensor(with_csr=exact)
        check(self.lib.s12_gemv_allreduce_async(self._h, C.byref(t), _ptr(bf16_in), _ptr(out), _stream(stream)),
              "s12_gemv_allreduce_async")

    @staticmethod
    def all_reduce_emulated(comms, srcs, dsts, stream=None) -> None:
        """All ranks of ``TPComm.local`` communicators in one cooperative launch (single-GPU tests)."""
        world = len(comms)
        arr = (C.c_void_p * world)(*[c._h for c in comms])
        ins = (C.c_void_p * world)(*[s.data_ptr() for s in srcs])
        outs = (C.c_void_p * world)(*[d.data_ptr() for d in dsts])
        check(comms[0].lib.s12_allreduce_f32_emulated_async(arr, world, ins, outs, srcs[0].numel(), _stream(stream)),
              "s12_allreduce_f32_emulated_async")

    def tp_argmax(self, logits: torch.Tensor, index_offset: int, result: torch.Tensor, stream=None) -> None:
        """Greedy tokens from this rank's rows of the output projection: fp32 [batch][n_local] -> int32 [batch]."""
        batch, n_local = (1, logits.numel()) if logits.dim() == 1 else logits.shape
        check(self.lib.s12_tp_argmax_async(self._h, _ptr(logits), n_local, index_offset, batch, _ptr(result), _stream(stream)),
              "s12_tp_argmax_async")

    def set_wait_limit_ms(self, ms: int) -> int:
        """How long a kernel waits for a peer before it gives up (default 2000 ms); returns the old limit."""
        old = self.lib.s12_comm_set_wait_limit_ms(self._h, int(ms))
        if old < 0:
            check(old, "s12_comm_set_wait_limit_ms")
        return old

    def reset(self) -> None:
        """After a call that gave up: zero this rank's receive areas and call counter (every rank calls it)."""
        check(self.lib.s12_comm_reset(self._h), "s12_comm_reset")

    def close(self) -> None:
        if self._h:
            self.lib.s12_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
