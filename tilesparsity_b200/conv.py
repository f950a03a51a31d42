"""Convolution on the masked GEMM without an im2col matrix.

The reference prunes conv kernels as [(kh*kw*cin), cout] matrices (img2col_forward,
Pruning/VGG/prune_algo.py:16-24) and runs the convolution in TensorFlow; its GEMM driver has no conv
path.  `ConvTWLayer` takes such a tile-wise sparse kernel and computes the stride-1, same-padded
convolution of an NHWC activation with it: the input is stored once per horizontal tap as padded
channel-major planes (ts_conv_pack_input), the masked GEMM gathers the rows of the virtual im2col
matrix out of them (ts_masked_conv), and the result is brought back to NHWC (ts_conv_unpack_output).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, lib
from .layer import TWLayer, _stream_ptr
from .tiles import TileSet


def geometry(B: int, H: int, W: int, kh: int, kw: int) -> dict:
    """Padded pixel space of a batch: Hp, Wp, m_padded (the GEMM's batch dimension), plane_ld."""
    hp, wp = C.c_int(), C.c_int()
    m, ld = C.c_int64(), C.c_int64()
    check(lib.ts_conv_geometry(B, H, W, kh, kw, C.byref(hp), C.byref(wp), C.byref(m), C.byref(ld)))
    return {"Hp": hp.value, "Wp": wp.value, "m_padded": m.value, "plane_ld": ld.value}


class ConvTWLayer:
    """A tile-wise sparse kh x kw convolution, weights HWIO [kh, kw, cin, cout] on the device."""

    def __init__(self, weights: torch.Tensor, tiles: TileSet, dtype=torch.bfloat16):
        if weights.dim() != 4:
            raise ValueError("weights must be HWIO [kh, kw, cin, cout]")
        self.kh, self.kw, self.cin, self.cout = (int(v) for v in weights.shape)
        if (tiles.K, tiles.N) != (self.kh * self.kw * self.cin, self.cout):
            raise ValueError("the tiles do not describe the kernel's [(kh*kw*cin), cout] matrix")
        self.dtype, self.device = dtype, weights.device
        self.layer = TWLayer(tiles, dtype, weights.device)
        self.layer.pack(weights.reshape(-1, self.cout).contiguous())
        with torch.cuda.device(self.device):
            check(lib.ts_layer_set_conv(self.layer._h, self.cin, self.kh, self.kw))

    def pack_input(self, x: torch.Tensor, planes: torch.Tensor | None = None):
        """NHWC activations [B, H, W, cin] -> (planes [kw, cin, plane_ld], geometry)."""
        if x.dim() != 4 or x.shape[3] != self.cin or x.dtype != self.dtype or not x.is_contiguous() or x.device != self.device:
            raise ValueError(f"x must be a contiguous [B, H, W, {self.cin}] {self.dtype} tensor on {self.device}")
        B, H, W, _ = (int(v) for v in x.shape)
        geo = geometry(B, H, W, self.kh, self.kw)
        if planes is None:
            planes = torch.empty((self.kw, self.cin, geo["plane_ld"]), dtype=self.dtype, device=self.device)
        if tuple(planes.shape) != (self.kw, self.cin, geo["plane_ld"]) or planes.dtype != self.dtype or not planes.is_contiguous():
            raise ValueError(f"planes must be a contiguous [{self.kw}, {self.cin}, {geo['plane_ld']}] tensor")
        with torch.cuda.device(self.device):
            check(lib.ts_conv_pack_input(C.c_void_p(x.data_ptr()), B, H, W, self.cin, self.kh, self.kw,
                                         C.c_void_p(planes.data_ptr()), geo["plane_ld"], _stream_ptr(self.device)))
        geo.update(B=B, H=H, W=W)
        return planes, geo

    def repack_input(self, ct_prev: torch.Tensor, geo: dict, planes: torch.Tensor | None = None):
        """The padded-space output Ct [cin, m_padded] of the previous convolution (same image size) as
        this layer's input planes: the chain conv -> conv stays channel-major, no NHWC round trip."""
        if ct_prev.dim() != 2 or ct_prev.shape[0] != self.cin or ct_prev.dtype != self.dtype or ct_prev.stride(1) != 1:
            raise ValueError(f"ct_prev must be a [{self.cin}, m_padded] {self.dtype} tensor with contiguous rows")
        g = geometry(geo["B"], geo["H"], geo["W"], self.kh, self.kw)
        if ct_prev.shape[1] < g["m_padded"] or g["Wp"] != geo["Wp"] or g["Hp"] != geo["Hp"]:
            raise ValueError("the previous output lives in another padded pixel space (different kernel size?)")
        if planes is None:
            planes = torch.empty((self.kw, self.cin, g["plane_ld"]), dtype=self.dtype, device=self.device)
        with torch.cuda.device(self.device):
            check(lib.ts_conv_repack(C.c_void_p(ct_prev.data_ptr()), ct_prev.stride(0), geo["B"], geo["H"], geo["W"], self.cin,
                                     self.kh, self.kw, C.c_void_p(planes.data_ptr()), g["plane_ld"], _stream_ptr(self.device)))
        g.update(B=geo["B"], H=geo["H"], W=geo["W"])
        return planes, g

    def masked_conv(self, planes: torch.Tensor, geo: dict, out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                    activation: str | None = None) -> torch.Tensor:
        """Ct [cout, m_padded] over the padded pixel space (pruned output channels stay as they are in `out`)."""
        if out is None:
            out = torch.zeros((self.cout, geo["m_padded"]), dtype=self.dtype, device=self.device)
        ep = _lib.Epilogue()
        ep.alpha, ep.beta = 1.0, 0.0
        if bias is not None:
            ep.bias_dev = bias.data_ptr()
        ep.activation = _lib.ACTIVATIONS[activation]
        with torch.cuda.device(self.device):
            check(lib.ts_masked_conv(self.layer._h, geo["B"], geo["H"], geo["W"], C.c_void_p(planes.data_ptr()),
                                     geo["plane_ld"], C.c_void_p(out.data_ptr()), out.stride(0), C.byref(ep),
                                     _stream_ptr(self.device)))
        return out

    def unpack_output(self, ct: torch.Tensor, geo: dict, y: torch.Tensor | None = None) -> torch.Tensor:
        if y is None:
            y = torch.empty((geo["B"], geo["H"], geo["W"], self.cout), dtype=self.dtype, device=self.device)
        with torch.cuda.device(self.device):
            check(lib.ts_conv_unpack_output(C.c_void_p(ct.data_ptr()), ct.stride(0), geo["B"], geo["H"], geo["W"], self.kh,
                                            self.kw, self.cout, C.c_void_p(y.data_ptr()), _stream_ptr(self.device)))
        return y

    def forward(self, x: torch.Tensor, bias: torch.Tensor | None = None, activation: str | None = None) -> torch.Tensor:
        """conv2d(x, W .* mask) (+ bias, activation) for NHWC x, stride 1, same padding; NHWC result."""
        planes, geo = self.pack_input(x)
        return self.unpack_output(self.masked_conv(planes, geo, bias=bias, activation=activation), geo)

    def algorithmic_bytes(self, B: int, H: int, W: int) -> int:
        """The NHWC input read once + packed weights + kept output channels written once + index lists."""
        st = self.layer.stats()
        kept = int(self.layer.tiles.n_counts().sum())
        px = B * H * W
        return px * self.cin * 2 + st["packed_bytes"] + px * kept * 2 + st["index_bytes"]

    def close(self) -> None:
        self.layer.close()
