"""Layer descriptors and model runners over the C-ABI operators.

Mirrors the reference's network layer (paths inside the APNN-TC project):

* ``Conv128LayerParam`` -- ``APNN-TC-nn/src/param.h:877-1083`` (shape math ``:915-924``),
* ``Fc128LayerParam`` -- ``param.h:219-385``, ``Out128LayerParam`` -- ``param.h:388-531``,
* the layer lists of ``APNN-TC-nn/src/alexnet.cu:43-81``, ``vgg.cu:49-127``, ``resnet18.cu:40-142``.

What a layer computes is fixed by ``LayerSpec`` below and restated on the CPU in
``tests/net_reference.py`` (the reference's programs never check a network output, so this
is project-defined): activations are ``a_bit`` levels in packed NHWC planes with a zero ring
for the next convolution, weights are 1-bit meaning -1/+1, every hidden layer requantises
through per-channel int32 thresholds (batch-norm folded on the host), pooling is a 2x2
maximum on the int32 value, a residual is the int32 value saved by an earlier layer, and
the output layer returns float logits (int32 values times a per-class scale plus a bias; or the
int32 values themselves), and the first layer reads the image at 8 bits (re-centred) unless
``first_bits`` is 0.  Channel counts are padded to multiples of 128 with
zero activations (padded output channels get thresholds no value reaches).

Everything here is host plumbing: every tensor operation is a call into ``libapnn_b200.so``.
"""
from __future__ import annotations

import ctypes
import os
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from . import _cabi
from .ops import _stream_ptr, make_epilogue

INT_MAX = 2**31 - 1


def pad128(c: int) -> int:
    return (c + 127) // 128 * 128


def padc(c: int, narrow: bool) -> int:
    """Stored channel count of a feature map: a multiple of 128, or 64 for maps of at most 64
    channels when the layers run on the tcgen05 path (64-byte swizzle rows)."""
    return 64 if (narrow and c <= 64) else pad128(c)


@dataclass
class LayerSpec:
    """One layer of a model list.  kind: 'conv' | 'fc' | 'out'."""
    name: str
    kind: str
    cin: int                      # real input channels / features
    cout: int                     # real output channels / features
    R: int = 1                    # filter size (conv)
    stride: int = 1
    pool: int = 1                 # 2 = 2x2 max pool after the conv
    save_residual: bool = False   # keep the int32 value for a later layer
    residual_from: Optional[str] = None   # name of the layer whose saved value is added
    src: Optional[str] = None     # input layer (default: the previous one)
    quantise: bool = True         # False: int32 output only (shortcut convs, logits)


@dataclass
class ModelSpec:
    name: str
    image_hw: int
    image_channels: int
    layers: List[LayerSpec]
    a_bit: int = 2
    w_bit: int = 1
    # The reference's higher-precision first and last layers (InConv128Layer / Out128Layer,
    # APNN-TC-nn/src/kernel.cuh:583-682, 397-447), as exact integer work plus one float affine:
    first_bits: int = 8        # 8: the image enters at 8 bits, re-centred (level - 128, padding = 0), times the
                               # -1/+1 filter on the int8 tensor-core path; 0: quantised to a_bit like a hidden map
    float_logits: bool = True  # the output layer returns float(value) * scale[c] + bias[c] instead of int32


def alexnet_spec(n_classes: int = 1000) -> ModelSpec:
    """APNN-TC-nn/src/alexnet.cu:43-81: 64c11s4+pool, 192c5+pool, 384c3, 256c3, 256c3+pool, 4096, 4096, out."""
    L = [
        LayerSpec("Conv1", "conv", 3, 64, 11, 4, pool=2),
        LayerSpec("Conv2", "conv", 64, 192, 5, 1, pool=2),
        LayerSpec("Conv3", "conv", 192, 384, 3),
        LayerSpec("Conv4", "conv", 384, 256, 3),
        LayerSpec("Conv5", "conv", 256, 256, 3, pool=2),
        LayerSpec("Fc1", "fc", 0, 4096),
        LayerSpec("Fc2", "fc", 4096, 4096),
        LayerSpec("Fout", "out", 4096, n_classes, quantise=False),
    ]
    return ModelSpec("alexnet", 224, 3, L)


def vgg_variant_spec(n_classes: int = 1000) -> ModelSpec:
    """The VGG-variant: 3x3 stacks of 128 / 256 / 512 channels with 2x2 pools, then 4096, 4096, out
    (layer plan of APNN-TC-nn/src/vgg.cu:49-127 with the 128/256/512 channel plan)."""
    L = [
        LayerSpec("Conv1", "conv", 3, 128, 3, 2, pool=2),
        LayerSpec("Conv2", "conv", 128, 256, 3), LayerSpec("Conv3", "conv", 256, 256, 3),
        LayerSpec("Conv4", "conv", 256, 256, 3, pool=2),
        LayerSpec("Conv5", "conv", 256, 512, 3), LayerSpec("Conv6", "conv", 512, 512, 3),
        LayerSpec("Conv7", "conv", 512, 512, 3, pool=2),
        LayerSpec("Conv8", "conv", 512, 512, 3), LayerSpec("Conv9", "conv", 512, 512, 3),
        LayerSpec("Conv10", "conv", 512, 512, 3, pool=2),
        LayerSpec("Fc1", "fc", 0, 4096), LayerSpec("Fc2", "fc", 4096, 4096),
        LayerSpec("Fout", "out", 4096, n_classes, quantise=False),
    ]
    return ModelSpec("vgg_variant", 224, 3, L)


def resnet18_spec(n_classes: int = 1000) -> ModelSpec:
    """APNN-TC-nn/src/resnet18.cu:40-142: 64c7s4, four stages of two basic blocks (64/128/256/512,
    stride 2 entering stages 2-4), FC 512, out.  The residual of a block is the saved int32 value
    of its input; where the shape changes it is a 1x1 stride-2 convolution of the block input."""
    L = [LayerSpec("Conv1", "conv", 3, 64, 7, 4, save_residual=True)]
    prev, cin = "Conv1", 64
    for stage, c in enumerate((64, 128, 256, 512), start=1):
        for blk in (1, 2):
            tag = f"L{stage}B{blk}"
            down = stage > 1 and blk == 1
            L.append(LayerSpec(tag + "C1", "conv", cin, c, 3, 2 if down else 1, src=prev))
            res = prev
            if down:
                L.append(LayerSpec(tag + "S", "conv", cin, c, 1, 2, src=prev, save_residual=True, quantise=False))
                res = tag + "S"
            L.append(LayerSpec(tag + "C2", "conv", c, c, 3, 1, src=tag + "C1", residual_from=res, save_residual=True))
            prev, cin = tag + "C2", c
    L += [LayerSpec("Fc1", "fc", 0, 512, src=prev), LayerSpec("Fout", "out", 512, n_classes, quantise=False)]
    return ModelSpec("resnet18", 224, 3, L)


MODELS = {"alexnet": alexnet_spec, "vgg_variant": vgg_variant_spec, "resnet18": resnet18_spec}


# ----------------------------------------------------------------------------- parameters (host, seeded)
@dataclass
class LayerParams:
    """Seeded random parameters of one layer in the library's layouts (numpy, host)."""
    weight_planes: np.ndarray     # conv: [1][COUTp][R][R][CINp/32]; fc/out: [1][Np][Kp/32]
    thresholds: Optional[np.ndarray]   # [COUTp][2^a_bit - 1] int32, or None when not quantised
    shape: Dict[str, int] = field(default_factory=dict)
    im2col_planes: Optional[np.ndarray] = None   # first layer only: [1][COUTp][PAD128(R*R*C)/32], k = (i*R+j)*C+c
    window_planes: Optional[np.ndarray] = None   # first layer only: the same filter for apnn_quantize_window_rows_i8
    affine: Optional[tuple] = None               # output layer with float logits: (scale, bias), float32 [COUTp]


def _pack_bits_msb(bits: np.ndarray) -> np.ndarray:
    """[..., K] of 0/1 -> [..., K/32] uint32, element k in bit 31 - k%32."""
    K = bits.shape[-1]
    by = np.packbits(bits.astype(np.uint8).reshape(*bits.shape[:-1], K // 32, 32), axis=-1, bitorder="big")
    return (by[..., 0].astype(np.uint32) << 24) | (by[..., 1].astype(np.uint32) << 16) | \
        (by[..., 2].astype(np.uint32) << 8) | by[..., 3].astype(np.uint32)


def _window_row_planes(bits: np.ndarray, narrow: bool) -> np.ndarray:
    """Filter bits [COUT][R][R][C] -> planes [1][COUT][kp/32] whose expansion (apnn_expand_planes) puts the
    weight of (i, j, c) at byte i*seg + j*C + c of a row, seg = R*C rounded up to 4: the layout of the rows
    apnn_quantize_window_rows_i8 writes.  Expansion puts packed element e of a 32-group at byte
    4*((31-e)&7) + ((31-e)>>3), so element e takes the weight meant for that byte."""
    cout, R, _, C = bits.shape
    seg = (R * C + 3) // 4 * 4
    kp = (R * seg + 63) // 64 * 64 if narrow else pad128(R * seg)
    rows = np.zeros((cout, kp), dtype=np.uint8)
    for i in range(R):
        rows[:, i * seg:i * seg + R * C] = bits[:, i].reshape(cout, R * C)
    f = 31 - np.arange(32)
    byte_of = 4 * (f & 7) + (f >> 3)
    packed_order = rows.reshape(cout, kp // 32, 32)[:, :, byte_of].reshape(cout, kp)
    return np.ascontiguousarray(_pack_bits_msb(packed_order)[None])


def _block_filter(im2col_planes: np.ndarray, R: int, stride: int, C: int, cpad: int) -> np.ndarray:
    """The first layer's +-1 filter (bits [1][COUT][PAD(R*R*C)/32], k = (i*R + j)*C + c) as the int8 rows of the
    stride-1 convolution over stride x stride pixel blocks (apnn_quantize_blocks_i8): [COUT][taps*taps*cpad] with
    the weight of image tap (ti, tj, c), ti = stride*(bi - halo) + di + pad, at block tap (bi, bj), byte
    (di*stride + dj)*C + c, and 0 where the filter does not reach."""
    words = np.ascontiguousarray(im2col_planes[0]).astype(np.uint32)
    cout = words.shape[0]
    shifts = np.arange(31, -1, -1, dtype=np.uint32)
    bits = ((words[:, :, None] >> shifts) & 1).reshape(cout, -1)[:, : R * R * C].reshape(cout, R, R, C).astype(np.int8)
    w = 2 * bits - 1
    pad = (R - 1) // 2
    halo = -(-pad // stride)
    taps = 2 * halo + 1
    out = np.zeros((cout, taps, taps, cpad), dtype=np.int8)
    for bi in range(taps):
        for di in range(stride):
            ti = stride * (bi - halo) + di + pad
            if not 0 <= ti < R:
                continue
            for bj in range(taps):
                for dj in range(stride):
                    tj = stride * (bj - halo) + dj + pad
                    if 0 <= tj < R:
                        ch = (di * stride + dj) * C
                        out[:, bi, bj, ch:ch + C] = w[:, ti, tj, :]
    return np.ascontiguousarray(out.reshape(cout, -1).view(np.uint8))


def window_rows_supported(W: int, C: int, R: int, stride: int, kp: int) -> bool:
    """The shapes apnn_quantize_window_rows_i8 takes (it returns APNN_ERR_UNSUPPORTED otherwise)."""
    pad, wc = (R - 1) // 2, W * C
    lpad = max(8, (pad * C + 3) // 4 * 4)
    rowlen = (lpad + wc + pad * C + 8 + 15) // 16 * 16
    Wo = (W - 1) // stride + 1
    return wc % 4 == 0 and R * rowlen <= 48 * 1024 and Wo * (kp // 16) <= 2048 and R * (wc // 4) <= 4096


def fold_thresholds(scale: np.ndarray, bias: np.ndarray, mu: float, sigma: float, out_bits: int) -> np.ndarray:
    """y = scale*(v-mu)/sigma + bias; level >= j exactly when y >= (j-0.5)*20/2^bits - 10 (the clip /
    round quantiser of APNN-TC-nn/src/kernel.cuh:29-44), so T[c][j-1] = ceil(mu + sigma*(edge_j - bias)/scale).
    Computed in double; the table is what host checker and kernels share."""
    nl = (1 << out_bits) - 1
    j = np.arange(1, nl + 1, dtype=np.float64)
    edge = (j - 0.5) * 20.0 / float(1 << out_bits) - 10.0
    t = mu + sigma * (edge[None, :] - bias.astype(np.float64)[:, None]) / scale.astype(np.float64)[:, None]
    return np.clip(np.ceil(t), -2**31, INT_MAX).astype(np.int64).astype(np.int32)


def make_params(spec: ModelSpec, seed: int = 0xA9117C + 5, image_hw: Optional[int] = None,
                narrow: bool = True) -> Dict[str, LayerParams]:
    """Random +-1 weights (uniform bits), BN scale U[0.5,1.5] and bias U[-1,1] folded to thresholds with
    mu = 0 and sigma = sqrt(3.5 * fan_in)/4 (variance of a +-1 x uniform-level dot product).
    narrow: store feature maps of at most 64 channels with 64 channels instead of 128 (the random
    draws cover real channels only, so both paddings hold the same network)."""
    rng = np.random.default_rng(seed)
    hw = image_hw or spec.image_hw
    out: Dict[str, LayerParams] = {}
    dims: Dict[str, tuple] = {}   # layer -> (H, W, C real) of its quantised output
    prev = None
    for ls in spec.layers:
        src = ls.src or prev
        if ls.kind == "conv":
            H, W, _ = dims[src] if src else (hw, hw, spec.image_channels)
            cinp, coutp = padc(ls.cin, narrow), padc(ls.cout, narrow)
            bits = np.zeros((coutp, ls.R, ls.R, cinp), dtype=np.uint8)
            bits[: ls.cout, :, :, : ls.cin] = rng.integers(0, 2, size=(ls.cout, ls.R, ls.R, ls.cin), dtype=np.uint8)
            planes = _pack_bits_msb(bits)[None]
            im2col = window = None
            if src is None:   # the same filter with the real channels only, laid out for the im2col first layer
                kp = (ls.R * ls.R * ls.cin + 63) // 64 * 64 if narrow else pad128(ls.R * ls.R * ls.cin)
                flat = np.zeros((coutp, kp), dtype=np.uint8)
                flat[:, : ls.R * ls.R * ls.cin] = bits[:, :, :, : ls.cin].reshape(coutp, -1)
                im2col = np.ascontiguousarray(_pack_bits_msb(flat)[None])
                window = _window_row_planes(bits[:, :, :, : ls.cin], narrow)
            Ho, Wo = (H - 1) // ls.stride + 1, (W - 1) // ls.stride + 1
            if ls.pool == 2:
                Ho, Wo = Ho // 2, Wo // 2
            fan_in = ls.R * ls.R * ls.cin
            dims[ls.name] = (Ho, Wo, ls.cout)
            shape = {"H": H, "W": W, "Ho": Ho, "Wo": Wo, "cinp": cinp, "coutp": coutp}
        else:
            if ls.kind == "fc" and ls.cin == 0:
                H, W, C = dims[src]
                K = H * W * padc(C, narrow)
                fan_in = H * W * C
                kbits = np.zeros((pad128(ls.cout), H, W, padc(C, narrow)), dtype=np.uint8)
                kbits[: ls.cout, :, :, :C] = rng.integers(0, 2, size=(ls.cout, H, W, C), dtype=np.uint8)
                kbits = kbits.reshape(pad128(ls.cout), K)
            else:
                K = pad128(ls.cin)
                fan_in = ls.cin
                kbits = np.zeros((pad128(ls.cout), K), dtype=np.uint8)
                kbits[: ls.cout, : ls.cin] = rng.integers(0, 2, size=(ls.cout, ls.cin), dtype=np.uint8)
            planes = _pack_bits_msb(kbits)[None]
            coutp = pad128(ls.cout)
            dims[ls.name] = (1, 1, ls.cout)
            shape = {"K": K, "coutp": coutp}
        thr = None
        affine = None
        if ls.kind == "out" and spec.float_logits:
            sc = np.zeros(coutp, dtype=np.float32)
            bi = np.zeros(coutp, dtype=np.float32)
            sc[: ls.cout] = rng.uniform(0.5, 1.5, ls.cout).astype(np.float32)
            bi[: ls.cout] = rng.uniform(-1.0, 1.0, ls.cout).astype(np.float32)
            affine = (sc, bi)
        if ls.quantise:
            scale = rng.uniform(0.5, 1.5, ls.cout).astype(np.float32)
            bias = rng.uniform(-1.0, 1.0, ls.cout).astype(np.float32)
            extra = 2.0 if ls.residual_from else 1.0
            # second moment of one input element: uniform a_bit levels, or the centred 8-bit image
            m2 = 5461.5 if (ls.kind == "conv" and src is None and spec.first_bits == 8) else 3.5
            sigma = math.sqrt(m2 * fan_in * extra) / 4.0
            thr = np.full((coutp, (1 << spec.a_bit) - 1), INT_MAX, dtype=np.int32)
            thr[: ls.cout] = fold_thresholds(scale, bias, 0.0, sigma, spec.a_bit)
        out[ls.name] = LayerParams(np.ascontiguousarray(planes), thr, shape, affine=affine)
        if ls.kind == "conv" and src is None:
            out[ls.name].im2col_planes = im2col
            out[ls.name].window_planes = window
        prev = ls.name
    return out


def value_bounds(spec: ModelSpec, params: Dict[str, LayerParams]) -> Dict[str, int]:
    """Largest magnitude the int32 value of each layer can take: (2^a - 1) * fan_in for +-1 weights and
    a-bit activations, plus the bound of the residual it adds.  A residual tensor whose bound is at most
    32767 can be stored as int16 without changing any result."""
    bound: Dict[str, int] = {}
    for ls in spec.layers:
        sh = params[ls.name].shape
        fan = sh["K"] if ls.kind != "conv" else ls.R * ls.R * ls.cin
        top = 128 if (ls is spec.layers[0] and spec.first_bits == 8) else (1 << spec.a_bit) - 1
        bound[ls.name] = top * fan + (bound[ls.residual_from] if ls.residual_from else 0)
    return bound


# ----------------------------------------------------------------------------- device runtime
def _dev_words(a: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).to(device)


class Network:
    """A model list bound to device buffers: weights (packed planes, and their int8 images for the
    tcgen05 path, expanded once), one output buffer per layer (packed planes inside the zero ring
    its consumers need), int32 residual buffers, and one shared int8 scratch for activations.

    ``forward(images)`` launches one packer and then, per layer, at most an activation expand and
    one contraction kernel, all on the current stream; ``capture()`` records that sequence in a
    CUDA graph for replay.
    """

    def __init__(self, spec: ModelSpec, batch: int, params: Optional[Dict[str, LayerParams]] = None,
                 device: Optional[torch.device] = None, image_hw: Optional[int] = None, use_tcgen05: bool = True):
        self.spec, self.batch = spec, batch
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.hw = image_hw or spec.image_hw
        self.params = params if params is not None else make_params(spec, image_hw=self.hw, narrow=use_tcgen05)
        self.use_tcgen05 = use_tcgen05
        self.L = _cabi.lib()
        self.by_name = {ls.name: ls for ls in spec.layers}
        a = spec.a_bit
        # ring each layer's output needs = the widest padding among its conv consumers
        prev = None
        self.src_of: Dict[str, Optional[str]] = {}
        halo: Dict[Optional[str], int] = {None: 0}
        for ls in spec.layers:
            src = ls.src or prev
            self.src_of[ls.name] = src
            halo.setdefault(ls.name, 0)
            if ls.kind == "conv":
                halo[src] = max(halo.get(src, 0), (ls.R - 1) // 2)
            prev = ls.name
        self.halo = halo
        B = batch
        cp = self.params[spec.layers[0].name].shape["cinp"]
        h0 = halo[None]
        self.out: Dict[str, torch.Tensor] = {}
        self.res: Dict[str, torch.Tensor] = {}
        self.w_planes: Dict[str, torch.Tensor] = {}
        self.w8: Dict[str, torch.Tensor] = {}
        self.thr: Dict[str, Optional[torch.Tensor]] = {}
        self.tc5_ok: Dict[str, bool] = {}
        self.first_im2col = None
        self.first_window_rows = False
        self.first_blocks = None   # (layer, Hb, Wb, block halo, block taps): the strided first layer on pixel blocks
        self.affine: Dict[str, tuple] = {}
        self.logit_acc = None
        if spec.first_bits not in (0, 8):
            raise ValueError("first_bits is 0 (a_bit levels) or 8 (centred 8-bit image)")
        if spec.first_bits == 8 and not use_tcgen05:
            raise ValueError("the 8-bit first layer runs on the tcgen05 path only")
        x8_bytes = 0
        for ls in spec.layers:
            p = self.params[ls.name]
            sh = p.shape
            self.w_planes[ls.name] = _dev_words(p.weight_planes, self.device)
            self.thr[ls.name] = _dev_words(p.thresholds, self.device) if p.thresholds is not None else None
            src = self.src_of[ls.name]
            if ls.kind == "conv":
                hh = halo[ls.name]
                if ls.quantise:
                    self.out[ls.name] = torch.zeros((a, B, sh["Ho"] + 2 * hh, sh["Wo"] + 2 * hh, sh["coutp"] // 32),
                                                    dtype=torch.int32, device=self.device)
                if ls.save_residual or not ls.quantise:
                    self.res[ls.name] = torch.zeros((B * sh["Ho"] * sh["Wo"], sh["coutp"]), dtype=torch.int32,
                                                    device=self.device)
                Hc, Wc = (sh["H"] - 1) // ls.stride + 1, (sh["W"] - 1) // ls.stride + 1
                pool_ok = not (ls.pool == 2 and (Hc % 2 or Wc % 2))
                ok = use_tcgen05 and ls.stride in (1, 2) and pool_ok
                if src is None and use_tcgen05 and pool_ok and p.im2col_planes is not None:
                    # first layer: windows gathered into channels, then a 1x1 convolution on tcgen05
                    kp = p.im2col_planes.shape[-1] * 32
                    wkp = p.window_planes.shape[-1] * 32
                    # whole-word gather where it covers the shape and does not widen the rows by more than a quarter
                    self.first_window_rows = (window_rows_supported(sh["W"], self.spec.image_channels, ls.R, ls.stride, wkp)
                                              and 4 * wkp <= 5 * kp)
                    if self.first_window_rows:
                        kp = wkp
                    self.first_im2col = (ls.name, Hc, Wc, kp)
                    self.w_planes[ls.name] = _dev_words(p.window_planes if self.first_window_rows else p.im2col_planes,
                                                        self.device)
                    x8_bytes = max(x8_bytes, B * Hc * Wc * kp)
                    ok = True
                    # A strided first layer on the centred 8-bit image: stride x stride pixel blocks as the "pixels" of
                    # a stride-1 convolution (apnn_quantize_blocks_i8), so the quantised image is written once, not
                    # once per window.
                    st, C0 = ls.stride, self.spec.image_channels
                    # Taken when the block convolution has 3 x 3 or 5 x 5 taps (7x7 and 11x11 filters at stride 4): those
                    # tap counts have straight-line MMA sequences in the flat convolution.
                    pad = (ls.R - 1) // 2
                    if (spec.first_bits == 8 and st >= 2 and st * st * C0 <= 64 and (st * C0) % 4 == 0 and pad <= 2 * st
                            and sh["H"] % st == 0 and sh["W"] % st == 0 and os.environ.get("APNN_FIRST_BLOCKS", "1") != "0"):
                        bh = -(-pad // st)
                        self.first_blocks = (ls.name, sh["H"] // st, sh["W"] // st, bh, 2 * bh + 1)
                self.tc5_ok[ls.name] = ok
                if not ok and sh["cinp"] % 128:
                    raise ValueError(f"{ls.name}: a {sh['cinp']}-channel input needs the tcgen05 path")
                if ok and not (self.first_im2col and self.first_im2col[0] == ls.name):
                    ih = halo[src]
                    x8_bytes = max(x8_bytes, B * (sh["H"] + 2 * ih) * (sh["W"] + 2 * ih) * sh["cinp"])
            else:
                self.tc5_ok[ls.name] = use_tcgen05
                if ls.quantise:
                    self.out[ls.name] = torch.zeros((a, B, sh["coutp"] // 32), dtype=torch.int32, device=self.device)
                else:
                    as_float = p.affine is not None
                    self.out[ls.name] = torch.zeros((B, sh["coutp"]), dtype=torch.float32 if as_float else torch.int32,
                                                    device=self.device)
                    if as_float:
                        self.affine[ls.name] = (torch.from_numpy(p.affine[0]).to(self.device),
                                                torch.from_numpy(p.affine[1]).to(self.device))
                        if not use_tcgen05:   # warp-level GEMM -> int32, then the affine as a pass of its own
                            self.logit_acc = torch.zeros((B, sh["coutp"]), dtype=torch.int32, device=self.device)
                if use_tcgen05:
                    x8_bytes = max(x8_bytes, B * sh["K"])
            if self.tc5_ok[ls.name]:
                wp = self.w_planes[ls.name]
                rows = wp.shape[1]
                k = int(np.prod(wp.shape[2:])) * 32
                w8 = torch.empty((rows, k), dtype=torch.uint8, device=self.device)
                _cabi.check(self.L.apnn_expand_planes(_stream_ptr(), wp.data_ptr(), w8.data_ptr(), rows, k, 1, 1),
                            "expand weights")
                self.w8[ls.name] = w8
                if self.first_blocks and self.first_blocks[0] == ls.name:
                    self.w8[ls.name] = torch.from_numpy(_block_filter(p.im2col_planes, ls.R, ls.stride,
                                                                      self.spec.image_channels, 64)).to(self.device)
                    _, Hb, Wb, bh, _ = self.first_blocks
                    self.xblocks = torch.zeros((B, Hb + 2 * bh, Wb + 2 * bh, 64), dtype=torch.uint8, device=self.device)
        if spec.first_bits == 8 and self.first_im2col is None:
            raise ValueError("the 8-bit first layer needs the gathered (im2col) form of the first convolution")
        # a quantised output feeds the next layers as int8 rows, written by the producing kernel's
        # epilogue, when producer and every consumer run on the tcgen05 path: no packed planes in
        # between and no expand pass
        # residual tensors are int16 where every value provably fits: |value| <= (2^a - 1) * fan_in
        # plus the bound of the residual it adds, and producer and readers run on the tcgen05 path
        self.res16: Dict[str, bool] = {}
        bound = value_bounds(spec, self.params)
        for ls in spec.layers:
            if ls.name in self.res:
                readers = [c.name for c in spec.layers if c.residual_from == ls.name]
                if (use_tcgen05 and self.tc5_ok[ls.name] and all(self.tc5_ok[r] for r in readers)
                        and bound[ls.name] <= 32767 and ls.quantise):
                    self.res[ls.name] = torch.zeros(self.res[ls.name].shape, dtype=torch.int16, device=self.device)
                    self.res16[ls.name] = True
        self.i8_out: Dict[str, bool] = {}
        for ls in spec.layers:
            users = [c.name for c in spec.layers if self.src_of[c.name] == ls.name]
            if use_tcgen05 and ls.quantise and users and self.tc5_ok[ls.name] and all(self.tc5_ok[u] for u in users):
                sh = self.params[ls.name].shape
                if ls.kind == "conv":
                    hh = halo[ls.name]
                    shape = (B, sh["Ho"] + 2 * hh, sh["Wo"] + 2 * hh, sh["coutp"])
                else:
                    shape = (B, sh["coutp"])
                self.out[ls.name] = torch.zeros(shape, dtype=torch.uint8, device=self.device)
                self.i8_out[ls.name] = True
        # pooled stride-1 layers whose output leaves as int8 rows run the (faster) flat convolution
        # unpooled into a scratch map and pool the level bytes afterwards: with ascending thresholds
        # the maximum of the levels is the level of the maximum.  (Fully connected layers with few
        # output tiles and a long K need nothing here: apnn_gemm_i8 splits K over CTA clusters.)
        self.split_pool: Dict[str, bool] = {}
        pool_bytes = 0
        for ls in spec.layers:
            if (ls.kind == "conv" and ls.pool == 2 and self.i8_out.get(ls.name, False) and not ls.save_residual
                    and ls.residual_from is None and (ls.stride == 1 or (self.first_im2col and self.first_im2col[0] == ls.name))):
                sh = self.params[ls.name].shape
                self.split_pool[ls.name] = True
                pool_bytes = max(pool_bytes, B * 2 * sh["Ho"] * 2 * sh["Wo"] * sh["coutp"])
        self.unpooled = torch.empty(max(pool_bytes, 16), dtype=torch.uint8, device=self.device)
        if self.first_im2col is None:
            self.image_planes = torch.zeros((a, B, self.hw + 2 * h0, self.hw + 2 * h0, cp // 32), dtype=torch.int32,
                                            device=self.device)
            self.image_levels = torch.zeros((a, B, self.hw, self.hw, cp // 32), dtype=torch.int32,
                                            device=self.device) if h0 else None
        self.x8 = torch.empty(max(x8_bytes, 256), dtype=torch.uint8, device=self.device)
        self.flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.graph = None
        self.static_images = None
        self.launches_per_forward = 0
        torch.cuda.synchronize(self.device)

    # -- one layer -------------------------------------------------------------------
    def levels_of(self, name: str) -> torch.Tensor:
        """Quantised output of a layer as levels [B, (H, W,) C] without its ring, whichever form it is stored in."""
        t, h = self.out[name], self.halo.get(name, 0)
        if self.i8_out.get(name, False):
            e = torch.arange(32, device=t.device)
            pos = 4 * ((31 - e) & 7) + ((31 - e) >> 3)      # byte of element e inside a group of 32 channels
            g = t.reshape(t.shape[:-1] + (t.shape[-1] // 32, 32))[..., pos].reshape(t.shape)
        else:
            shifts = torch.arange(31, -1, -1, device=t.device, dtype=torch.int32)
            bitsel = (t.unsqueeze(-1) >> shifts) & 1                     # [a, ..., C/32, 32]
            g = sum((bitsel[b].to(torch.uint8) << b) for b in range(t.shape[0])).reshape(t.shape[1:-1] + (t.shape[-1] * 32,))
        return g[:, h:g.shape[1] - h, h:g.shape[2] - h] if (h and g.dim() == 4) else g

    def _input_of(self, name: str) -> torch.Tensor:
        src = self.src_of[name]
        if src is None:
            return None if self.first_im2col else self.image_planes   # the im2col first layer reads self.x8
        return self.out[src]

    def _epilogue(self, ls: LayerSpec, conv: bool):
        if ls.name in self.affine:
            sc, bi = self.affine[ls.name]
            return make_epilogue("float", affine_scale=sc, affine_bias=bi)
        mode = "thresholds" if ls.quantise else "int32"
        res_in = self.res[ls.residual_from] if ls.residual_from else None
        res_out = self.res.get(ls.name) if (ls.save_residual and ls.quantise) else None
        r16 = (1 if (ls.residual_from and self.res16.get(ls.residual_from, False)) else 0) | \
              (2 if (res_out is not None and self.res16.get(ls.name, False)) else 0)
        split = self.split_pool.get(ls.name, False)
        return make_epilogue(mode, self.spec.a_bit if ls.quantise else 0, signed="none",
                             pool="max" if (ls.pool == 2 and not split) else "none",
                             out_halo=self.halo[ls.name] if (conv and not split) else 0,
                             in_halo=self.halo[self.src_of[ls.name]] if conv else 0, thresholds=self.thr[ls.name],
                             residual_in=res_in, residual_out=res_out, out_i8=self.i8_out.get(ls.name, False),
                             residual_i16=r16)

    def _run_conv(self, ls: LayerSpec) -> int:
        sh = self.params[ls.name].shape
        X = self._input_of(ls.name)
        a, B = self.spec.a_bit, self.batch
        epi = self._epilogue(ls, True)
        out = self.out[ls.name] if ls.quantise else self.res[ls.name]
        s = _stream_ptr()
        if self.split_pool.get(ls.name, False):
            final, out = out, self.unpooled
            n = self._launch_conv(ls, sh, X, a, B, epi, out, s)
            _cabi.check(self.L.apnn_maxpool2x2_i8(s, out.data_ptr(), final.data_ptr(), B, 2 * sh["Ho"], 2 * sh["Wo"],
                                                  sh["coutp"], 0, self.halo[ls.name]), "apnn_maxpool2x2_i8 " + ls.name)
            return n + 1
        return self._launch_conv(ls, sh, X, a, B, epi, out, s)

    def _launch_conv(self, ls, sh, X, a, B, epi, out, s) -> int:
        if self.first_blocks and self.first_blocks[0] == ls.name:
            _, Hb, Wb, bh, taps = self.first_blocks
            epi.in_halo = bh
            # filter bytes -1 / 0 / +1 (bit 0), centred signed image bytes (bit 1)
            _cabi.check(self.L.apnn_conv2d_i8(s, self.w8[ls.name].data_ptr(), self.xblocks.data_ptr(), out.data_ptr(), B,
                                              Hb, Wb, 64, sh["coutp"], taps, 1, 3, ctypes.byref(epi), self.flag.data_ptr()),
                        "apnn_conv2d_i8 " + ls.name)
            return 1
        if self.first_im2col and self.first_im2col[0] == ls.name:
            _, Hc, Wc, kp = self.first_im2col
            epi.in_halo = 0
            signs = 3 if self.spec.first_bits == 8 else 1   # bit 0: -1/+1 filter bytes; bit 1: centred (signed) image bytes
            _cabi.check(self.L.apnn_conv2d_i8(s, self.w8[ls.name].data_ptr(), self.x8.data_ptr(), out.data_ptr(), B,
                                              Hc, Wc, kp, sh["coutp"], 1, 1, signs, ctypes.byref(epi), self.flag.data_ptr()),
                        "apnn_conv2d_i8 " + ls.name)
            return 1
        if self.tc5_ok[ls.name]:
            n, x8 = 1, X
            if not self.i8_out.get(self.src_of[ls.name], False):
                rows = X.shape[1] * X.shape[2] * X.shape[3]
                _cabi.check(self.L.apnn_expand_planes(s, X.data_ptr(), self.x8.data_ptr(), rows, sh["cinp"], a, 0), "expand")
                n, x8 = 2, self.x8
            _cabi.check(self.L.apnn_conv2d_i8(s, self.w8[ls.name].data_ptr(), x8.data_ptr(), out.data_ptr(), B,
                                              sh["H"], sh["W"], sh["cinp"], sh["coutp"], ls.R, ls.stride, 1,
                                              ctypes.byref(epi), self.flag.data_ptr()), "apnn_conv2d_i8 " + ls.name)
            return n
        epi.signed_operand = _cabi.SIGN_W
        _cabi.check(self.L.apnn_conv2d_ex(s, _cabi.ALGO_IMMA, 1, a, self.w_planes[ls.name].data_ptr(), X.data_ptr(),
                                          out.data_ptr(), B, sh["H"], sh["W"], sh["cinp"], sh["coutp"], ls.R, ls.stride,
                                          ctypes.byref(epi), None, 0), "apnn_conv2d_ex " + ls.name)
        return 1

    def _run_fc(self, ls: LayerSpec) -> int:
        sh = self.params[ls.name].shape
        X = self._input_of(ls.name)       # [a][B][...] packed, no ring
        a, B, K, N = self.spec.a_bit, self.batch, sh["K"], sh["coutp"]
        epi = self._epilogue(ls, False)
        out = self.out[ls.name]
        s = _stream_ptr()
        if self.tc5_ok[ls.name]:
            n, x8 = 1, X
            if not self.i8_out.get(self.src_of[ls.name], False):
                _cabi.check(self.L.apnn_expand_planes(s, X.data_ptr(), self.x8.data_ptr(), B, K, a, 0), "expand")
                n, x8 = 2, self.x8
            _cabi.check(self.L.apnn_gemm_i8(s, x8.data_ptr(), self.w8[ls.name].data_ptr(), out.data_ptr(), B, N, K,
                                            0, 1, ctypes.byref(epi), self.flag.data_ptr()), "apnn_gemm_i8 " + ls.name)
            return n
        if ls.name in self.affine:
            plain = make_epilogue("int32", signed="x")
            _cabi.check(self.L.apnn_gemm_ex(s, _cabi.ALGO_IMMA, a, 1, X.data_ptr(), self.w_planes[ls.name].data_ptr(),
                                            self.logit_acc.data_ptr(), B, N, K, ctypes.byref(plain), None, 0),
                        "apnn_gemm_ex " + ls.name)
            _cabi.check(self.L.apnn_requantize_i32(s, self.logit_acc.data_ptr(), out.data_ptr(), B, N, ctypes.byref(epi)),
                        "apnn_requantize_i32 " + ls.name)
            return 2
        epi.signed_operand = _cabi.SIGN_X
        _cabi.check(self.L.apnn_gemm_ex(s, _cabi.ALGO_IMMA, a, 1, X.data_ptr(), self.w_planes[ls.name].data_ptr(),
                                        out.data_ptr(), B, N, K, ctypes.byref(epi), None, 0), "apnn_gemm_ex " + ls.name)
        return 1

    # -- whole model -----------------------------------------------------------------
    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """images: float32 [B, H, W, C] on the device.  Returns the logits [B, PAD128(classes)]: float32 with
        ``float_logits`` (the default), else the int32 values."""
        a = self.spec.a_bit
        s = _stream_ptr()
        rows = self.batch * self.hw * self.hw
        n = 1
        h0 = self.halo[None]
        if self.first_blocks:
            first = self.by_name[self.first_blocks[0]]
            _cabi.check(self.L.apnn_quantize_blocks_i8(s, images.data_ptr(), self.xblocks.data_ptr(), self.batch, self.hw,
                                                       self.hw, self.spec.image_channels, first.stride,
                                                       8 | _cabi.QUANT_CENTRED, self.first_blocks[3], 64),
                        "first-layer block quantiser")
        elif self.first_im2col:
            # quantise + gather the first layer's windows straight into the int8 operand buffer
            first = self.by_name[self.first_im2col[0]]
            gather = self.L.apnn_quantize_window_rows_i8 if self.first_window_rows else self.L.apnn_quantize_im2col_i8
            bits = (8 | _cabi.QUANT_CENTRED) if self.spec.first_bits == 8 else a
            _cabi.check(gather(s, images.data_ptr(), self.x8.data_ptr(), self.batch, self.hw, self.hw,
                               self.spec.image_channels, first.R, first.stride, bits, self.first_im2col[3]),
                        "first-layer gather")
        else:
            target = self.image_levels if h0 else self.image_planes
            _cabi.check(self.L.apnn_quantize_pack(s, images.data_ptr(), target.data_ptr(), rows,
                                                  self.spec.image_channels, a), "apnn_quantize_pack")
            if h0:
                # place the packed image inside its zero ring (device-side strided copy)
                self.image_planes[:, :, h0:-h0, h0:-h0].copy_(self.image_levels)
                n += 1
        for ls in self.spec.layers:
            n += self._run_conv(ls) if ls.kind == "conv" else self._run_fc(ls)
        self.launches_per_forward = n
        return self.out[self.spec.layers[-1].name]

    def capture(self, images: torch.Tensor) -> None:
        """Record forward(images) in a CUDA graph; ``replay()`` reruns it on the same buffers."""
        self.static_images = images
        self.forward(images)  # warm-up: function attributes, descriptor caches
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream(device=self.device)
        st.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                self.forward(images)
        torch.cuda.synchronize(self.device)
        self.graph = g

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out[self.spec.layers[-1].name]

    def check(self) -> None:
        """Synchronise and raise if a tcgen05 kernel gave up on a bounded wait."""
        torch.cuda.synchronize(self.device)
        if int(self.flag.item()) != 0:
            raise _cabi.ApnnError(7, "a bounded device-side wait expired")
