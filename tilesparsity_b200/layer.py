"""Python operator surface over the C ABI: a tile-wise sparse layer and its masked GEMM.

`TWLayer` owns one `ts_layer_t` handle (index lists, packed weights, schedules on the device).
`masked_gemm` is the whole-layer replacement of the reference's Stream_Gemm_NN
(StreamMaskedGEMM/perf/basic_nn.cu:378-445) in the reference's own K-major layout; `masked_linear`
is the op the reference's model code expresses as `matmul(x, kernel * mask)`
(Pruning/BERT/utils/modeling.py:992-1007) for row-major activations.  PyTorch supplies device
memory and streams only; all arithmetic runs in libtilesparse's CUDA kernels.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .tiles import TileSet, tiles_from_lists, tiles_from_mask

_TS_DTYPE = {torch.float16: _lib.TS_DTYPE_F16, torch.bfloat16: _lib.TS_DTYPE_BF16,
             torch.float32: _lib.TS_DTYPE_F32}


def _stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _i32(a: np.ndarray):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


class TWLayer:
    """One tile-wise sparse weight matrix W[K, N] resident on a B200."""

    def __init__(self, tiles: TileSet, dtype=torch.float16, device=None):
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("compute dtype must be torch.float16 or torch.bfloat16")
        if not torch.cuda.is_available():
            raise RuntimeError("TWLayer needs a CUDA device (there is no CPU fallback)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dtype = dtype
        self.tiles = tiles
        self.K, self.N, self.G = tiles.K, tiles.N, tiles.G
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.ts_layer_create(C.byref(self._h), self.K, self.N, self.G, _TS_DTYPE[dtype]))
        self.retile(tiles)

    def retile(self, tiles: TileSet) -> None:
        """Installs another tile structure of the same [K, N] matrix (ts_layer_set_tiles); the packed
        weights are dropped, call `pack` again."""
        if (tiles.K, tiles.N) != (self.K, self.N) or tiles.G > self.G:
            raise ValueError("the new tiles describe another matrix")
        self.tiles = tiles
        with torch.cuda.device(self.device):
            self._kp, kp = _i32(tiles.tile_k_ptr)
            self._kk, kk = _i32(tiles.kept_k)
            self._np, npp = _i32(tiles.tile_n_ptr)
            self._nn, nn = _i32(tiles.kept_n)
            check(lib.ts_layer_set_tiles(self._h, tiles.n_tiles, kp, kk, npp, nn, _lib.TS_INDEX_ABSOLUTE))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_lists(cls, W: torch.Tensor, kept_k_lists, col_mask=None, G: int = 128, dtype=torch.float16):
        """W [K, N] on the device, per-tile kept-row lists, global column mask."""
        K, N = W.shape
        layer = cls(tiles_from_lists(K, N, G, kept_k_lists, col_mask), dtype, W.device)
        layer.pack(W)
        return layer

    @classmethod
    def from_mask(cls, W: torch.Tensor, mask, G: int = 128, col_mask=None, dtype=torch.float16):
        """W [K, N] on the device and a tile-wise 0/1 mask (NumPy or tensor) of the same shape."""
        if isinstance(mask, torch.Tensor):
            mask = mask.detach().cpu().numpy()
        if isinstance(col_mask, torch.Tensor):
            col_mask = col_mask.detach().cpu().numpy()
        layer = cls(tiles_from_mask(mask, G, col_mask), dtype, W.device)
        layer.pack(W)
        return layer

    @classmethod
    def grouped(cls, Ws, tile_sets, dtype=torch.float16):
        """Several independent tile-wise sparse layers as ONE layer, so that one launch computes all of
        them: the weights become a block-structured [sum K, sum N] matrix whose tile t of layer l keeps
        the rows (K offset of l) + kept rows, the activations are stacked [sum K][M] (layer l at row
        offset k_off[l]) and the outputs [sum N][M] (layer l at row offset n_off[l]).  Nothing in the
        kernel is special-cased: units of all layers share one schedule, and the start and end of the
        individual GEMMs overlap.  The layers must not depend on each other's outputs.
        Returns (layer, k_off, n_off); the dense block matrix exists only while the weights are packed."""
        if not Ws or len(Ws) != len(tile_sets):
            raise ValueError("one weight matrix per tile set")
        G = tile_sets[0].G
        dev = Ws[0].device
        k_off = np.concatenate([[0], np.cumsum([ts.K for ts in tile_sets])]).astype(np.int64)
        n_off = np.concatenate([[0], np.cumsum([ts.N for ts in tile_sets])]).astype(np.int64)
        lists, col_masks = [], []
        for l, ts in enumerate(tile_sets):
            if ts.G != G or (ts.N % G) != 0 and l + 1 < len(tile_sets):
                raise ValueError("layers must share G, and every layer but the last needs N divisible by G")
            lists += [(ts.tile_rows(t) + k_off[l]).astype(np.int32) for t in range(ts.n_tiles)]
            col_masks.append(ts.col_mask())
        col_mask = np.concatenate(col_masks)
        if not col_mask.all():
            raise ValueError("grouped layers with pruned columns are not supported")
        W_all = torch.zeros((int(k_off[-1]), int(n_off[-1])), dtype=Ws[0].dtype, device=dev)
        for l, W in enumerate(Ws):
            W_all[k_off[l]:k_off[l + 1], n_off[l]:n_off[l + 1]] = W
        layer = cls(tiles_from_lists(int(k_off[-1]), int(n_off[-1]), G, lists), dtype, dev)
        layer.pack(W_all)
        return layer, k_off, n_off

    def pack(self, W: torch.Tensor) -> None:
        if W.device != self.device or W.dim() != 2 or tuple(W.shape) != (self.K, self.N):
            raise ValueError(f"W must be a [{self.K}, {self.N}] tensor on {self.device}")
        if W.dtype not in _TS_DTYPE or W.stride(1) != 1:
            raise ValueError("W must be fp32/fp16/bf16 with contiguous rows")
        with torch.cuda.device(self.device):
            check(lib.ts_layer_pack_weights(self._h, C.c_void_p(W.data_ptr()), W.stride(0), _TS_DTYPE[W.dtype],
                                            _stream_ptr(self.device)))

    def set_unit_rows(self, unit_rows: int) -> None:
        """Pins the kernel variant (work units of at most 128 or 256 batch rows); 0 = automatic."""
        with torch.cuda.device(self.device):
            check(lib.ts_layer_set_unit_rows(self._h, int(unit_rows)))

    def set_split_k(self, enabled: bool) -> None:
        """Allows (default) or forbids split-K units: a tile with a long chain of K blocks cut into ranges
        that run as units of their own, their fp32 partial sums added up by a second kernel."""
        check(lib.ts_layer_set_split_k(self._h, 1 if enabled else 0))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            lib.ts_layer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ queries
    def packed_weights(self) -> torch.Tensor:
        """[n_tiles*128, ldw] host copy of the compacted weights (row t*128+j = kept column j of tile t)."""
        rows, ldw = C.c_int64(), C.c_int64()
        check(lib.ts_layer_get_packed(self._h, None, C.byref(rows), C.byref(ldw)))
        out = torch.empty((rows.value, ldw.value), dtype=self.dtype)
        with torch.cuda.device(self.device):
            check(lib.ts_layer_get_packed(self._h, C.c_void_p(out.data_ptr()), C.byref(rows), C.byref(ldw)))
        return out

    def stats(self) -> dict:
        f, pb, ib = C.c_int64(), C.c_int64(), C.c_int64()
        nt, mk = C.c_int(), C.c_int()
        check(lib.ts_layer_stats(self._h, C.byref(f), C.byref(pb), C.byref(ib), C.byref(nt), C.byref(mk)))
        return {"kept_flops_per_row": f.value, "packed_bytes": pb.value, "index_bytes": ib.value,
                "n_tiles": nt.value, "max_kept_k": mk.value}

    def schedule_stats(self, M: int) -> dict:
        n, u = C.c_int(), C.c_int()
        with torch.cuda.device(self.device):
            check(lib.ts_layer_schedule_stats(self._h, M, C.byref(n), None, C.byref(u)))
            cost = np.zeros(n.value, dtype=np.float32)
            check(lib.ts_layer_schedule_stats(self._h, M, C.byref(n), cost.ctypes.data_as(C.POINTER(C.c_float)),
                                              C.byref(u)))
        mean = float(cost.mean()) if len(cost) else 0.0
        return {"n_ctas": n.value, "n_units": u.value, "cta_cost": cost,
                "makespan": float(cost.max()) if len(cost) else 0.0, "mean": mean,
                "balance": (mean / float(cost.max())) if len(cost) and cost.max() > 0 else 1.0}

    def algorithmic_bytes(self, M: int) -> int:
        """A read once + packed W + kept C written once + index lists (per call, beta = 0)."""
        st = self.stats()
        kept_cols = int(self.tiles.n_counts().sum())
        return M * self.K * 2 + st["packed_bytes"] + M * kept_cols * 2 + st["index_bytes"]

    # ------------------------------------------------------------------ compute
    def masked_gemm(self, At: torch.Tensor, out: torch.Tensor | None = None, alpha: float = 1.0,
                    beta: float = 0.0, simt: bool = False, bias: torch.Tensor | None = None,
                    activation: str | None = None, peers=None, multicast: int | None = None) -> torch.Tensor:
        """Ct[N, M] = act(alpha * (W .* mask)^T @ At[K, M] + beta * Ct + bias[:, None]), kept columns only.

        At is the reference's activation layout: [K, M] with M contiguous.  Without `out` a zeroed
        [N, M] tensor is allocated, so pruned columns read as zero.  bias is fp32 [N]; activation is
        None, "relu" or "gelu"; peers are raw device addresses of further [N, M] buffers (same row
        pitch as `out`) that receive the same rows, e.g. the other GPUs' copies of a sharded output;
        `multicast` is instead the NVSwitch multicast address of `out` (the switch delivers every
        store to all GPUs' copies, this one included).
        """
        if At.dim() != 2 or At.shape[0] != self.K or At.dtype != self.dtype or At.device != self.device:
            raise ValueError(f"At must be a [{self.K}, M] {self.dtype} tensor on {self.device}")
        if At.stride(1) != 1:
            raise ValueError("At must have M contiguous")
        M = At.shape[1]
        if out is None:
            out = torch.zeros((self.N, M), dtype=self.dtype, device=self.device)
        if tuple(out.shape) != (self.N, M) or out.dtype != self.dtype or out.stride(1) != 1 or out.device != self.device:
            raise ValueError(f"out must be a [{self.N}, {M}] {self.dtype} tensor with M contiguous")
        with torch.cuda.device(self.device):
            if simt:
                if bias is not None or activation or peers:
                    raise ValueError("the CUDA-core twin has no fused epilogue")
                check(lib.ts_masked_gemm_simt(self._h, M, C.c_void_p(At.data_ptr()), At.stride(0),
                                              C.c_void_p(out.data_ptr()), out.stride(0), alpha, beta,
                                              _stream_ptr(self.device)))
                return out
            ep = _lib.Epilogue()
            ep.alpha, ep.beta = alpha, beta
            if bias is not None:
                if bias.dtype != torch.float32 or bias.numel() != self.N or bias.device != self.device or not bias.is_contiguous():
                    raise ValueError(f"bias must be a contiguous fp32 [{self.N}] tensor on {self.device}")
                ep.bias_dev = bias.data_ptr()
            if activation not in _lib.ACTIVATIONS:
                raise ValueError(f"unknown activation {activation!r}")
            ep.activation = _lib.ACTIVATIONS[activation]
            peers = list(peers or [])
            if len(peers) > 7:
                raise ValueError("at most 7 peer buffers")
            ep.n_peers = len(peers)
            for i, p in enumerate(peers):
                ep.peer_ct[i] = int(p)
            if multicast:
                # the multicast address of `out`: one multimem store per piece reaches every GPU's copy
                ep.multicast_ct = int(multicast)
            check(lib.ts_masked_gemm_ex(self._h, M, C.c_void_p(At.data_ptr()), At.stride(0), C.c_void_p(out.data_ptr()),
                                        out.stride(0), C.byref(ep), _stream_ptr(self.device)))
        return out

    def masked_gemm_host(self, At_host: torch.Tensor, Ct_host: torch.Tensor, alpha: float = 1.0,
                         beta: float = 0.0, wait: bool = True) -> torch.Tensor:
        """Host-buffer variant: contiguous H2D copy, GEMM, contiguous D2H copy (one C-ABI call).
        With wait=False the call returns once everything is queued; `host_wait()` then orders the
        current stream after the arrival of the output, and Ct_host is valid once that stream has
        been synchronised."""
        if At_host.is_cuda or Ct_host.is_cuda:
            raise ValueError("masked_gemm_host takes host tensors")
        if At_host.dtype != self.dtype or Ct_host.dtype != self.dtype:
            raise ValueError(f"host tensors must be {self.dtype}")
        if not (At_host.is_contiguous() and Ct_host.is_contiguous()):
            raise ValueError("host tensors must be contiguous")
        M = At_host.shape[1]
        if tuple(At_host.shape) != (self.K, M) or tuple(Ct_host.shape) != (self.N, M):
            raise ValueError("shape mismatch")
        with torch.cuda.device(self.device):
            fn = lib.ts_masked_gemm_host if wait else lib.ts_masked_gemm_host_async
            check(fn(self._h, M, C.c_void_p(At_host.data_ptr()), C.c_void_p(Ct_host.data_ptr()), alpha, beta,
                     _stream_ptr(self.device)))
        return Ct_host

    def host_wait(self) -> None:
        """Makes the current stream wait for this layer's latest masked_gemm_host(wait=False)."""
        with torch.cuda.device(self.device):
            check(lib.ts_masked_gemm_host_wait(self._h, _stream_ptr(self.device)))

    def check(self) -> None:
        """Raises if a kernel of this layer recorded an error (synchronises the current stream)."""
        with torch.cuda.device(self.device):
            check(lib.ts_layer_check(self._h, _stream_ptr(self.device)))


class TEWLayer:
    """A TEW layer: tile-wise part on the tensor cores plus the element-wise residual as a sparse term.

    Built from the output of `build_mask("tw1m" | "tw2m", ..., want_residual=True)`: `tiles` is the
    tile-wise structure, `residual` a bool [K, N] CUDA tensor marking the extra elements
    (Pruning/VGG/prune_algo.py:171-175 adds them to the dense mask).
    """

    def __init__(self, W: torch.Tensor, tiles: TileSet, residual: torch.Tensor, dtype=torch.float16):
        self.tw = TWLayer(tiles, dtype, W.device)
        self.tw.pack(W)
        self.dtype, self.device, self.K, self.N = dtype, W.device, tiles.K, tiles.N
        nz = residual.t().nonzero()                       # sorted by (n, k)
        cols, rows = nz[:, 0], nz[:, 1]
        self.nnz = int(nz.shape[0])
        counts = torch.bincount(cols, minlength=self.N)
        self.col_ptr = torch.zeros(self.N + 1, dtype=torch.int32, device=W.device)
        self.col_ptr[1:] = torch.cumsum(counts, 0).to(torch.int32)
        self.row_idx = rows.to(torch.int32).contiguous()
        self.val = W[rows, cols].to(dtype).contiguous()
        written = torch.zeros(self.N, dtype=torch.uint8, device=W.device)
        written[torch.from_numpy(tiles.kept_n.astype(np.int64)).to(W.device)] = 1
        self.col_written = written

    def masked_gemm(self, At: torch.Tensor, out: torch.Tensor | None = None, alpha: float = 1.0) -> torch.Tensor:
        """Ct[N, M] = alpha * (W .* mask_tew)^T @ At[K, M]."""
        Ct = self.tw.masked_gemm(At, out=out, alpha=alpha)
        M = At.shape[1]
        if self.nnz:
            with torch.cuda.device(self.device):
                check(lib.ts_residual_gemm(_TS_DTYPE[self.dtype], M, self.N, C.c_void_p(self.col_ptr.data_ptr()),
                                           C.c_void_p(self.row_idx.data_ptr()), C.c_void_p(self.val.data_ptr()),
                                           C.c_void_p(self.col_written.data_ptr()), C.c_void_p(At.data_ptr()),
                                           At.stride(0), C.c_void_p(Ct.data_ptr()), Ct.stride(0), alpha,
                                           _stream_ptr(self.device)))
        return Ct

    def close(self) -> None:
        self.tw.close()


def transpose16(x: torch.Tensor) -> torch.Tensor:
    """[R, C] 16-bit tensor -> its transpose [C, R], materialised by the library's kernel."""
    if x.dim() != 2 or x.element_size() != 2 or x.stride(1) != 1 or not x.is_cuda:
        raise ValueError("transpose16 takes a 2-D 16-bit CUDA tensor with contiguous rows")
    R, Cc = x.shape
    out = torch.empty((Cc, R), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.ts_transpose16(C.c_void_p(x.data_ptr()), x.stride(0), C.c_void_p(out.data_ptr()), out.stride(0),
                                 R, Cc, _stream_ptr(x.device)))
    return out


def masked_linear(A: torch.Tensor, layer: TWLayer, transpose_out: bool = True) -> torch.Tensor:
    """`A @ (W * mask)` for row-major activations A[M, K]  (mask_dense, modeling.py:992-1007, minus bias).

    A is transposed to the K-major layout on the device first (an extra pass the K-major entry point
    `TWLayer.masked_gemm` does not pay).  Returns C[M, N], or Ct[N, M] with transpose_out=False.
    """
    Ct = layer.masked_gemm(transpose16(A))
    return transpose16(Ct) if transpose_out else Ct


def masked_matmul(A: torch.Tensor, W: torch.Tensor, kept_k_lists, col_mask=None, G: int = 128) -> torch.Tensor:
    """Functional form: activations A[M, K], weights W[K, N], per-tile kept-K-row index lists and a
    global column mask.  Packs W on every call; keep a `TWLayer` when the weights are reused."""
    layer = TWLayer.from_lists(W, kept_k_lists, col_mask, G, A.dtype)
    try:
        return masked_linear(A, layer)
    finally:
        torch.cuda.current_stream(A.device).synchronize()
        layer.close()
