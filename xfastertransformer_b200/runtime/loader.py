"""Checkpoint IO: raw ``.bin`` tensors, TP/EP slicing at load, quantise-at-load.

On-disk contract (reference converters, e.g. ``src/xfastertransformer/tools/llama_convert.py:33-45,
177-200``; loader ``src/utils/weight_util.h:71-218``): headerless little-endian C-order tensors, linear
weights stored ``[in, out]``, element type = ``weight_data_type`` of ``config.ini``.

Device contract of this engine: every linear weight lives as ``[out, in]`` (K contiguous) so
that both tcgen05 operands are K-major and one TMA box covers 64 K-elements (a 128-byte swizzle
row).  Slicing happens before the transpose, straight from a memory-mapped file, so a rank only
touches its own bytes; the reference reads whole tensors on every rank
(``src/layers/decoder_block.h:495-827``).

``XFT_FAKE_MODEL=1`` zero-fills like the reference (``weight_util.h:76-82``); ``=2`` draws
N(0, 0.02) on the device (synthetic benchmarks: no files needed beyond config.ini).
"""
from __future__ import annotations

import os
import zlib
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import reference as R
from ..utils.flags import Env

_NP = {"fp32": np.float32, "fp16": np.float16, "bf16": np.uint16, "int8": np.int8, "uint8": np.uint8,
       "fp8_e4m3": np.uint8, "int32": np.int32}
_TORCH = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def write_bin(path: str, t: torch.Tensor, dtype: str) -> None:
    """Write `t` as a headerless .bin of element type `dtype` (fp32|fp16|bf16|int8|uint8|fp8_e4m3)."""
    t = t.detach().cpu().contiguous()
    if dtype == "bf16":
        arr = t.to(torch.bfloat16).view(torch.int16).numpy()
    elif dtype == "fp8_e4m3":
        arr = t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    elif dtype in ("fp32", "fp16"):
        arr = t.to(_TORCH[dtype]).numpy()
    else:
        arr = t.numpy().astype(_NP[dtype])
    arr.tofile(path)


def read_bin(path: str, dtype: str, shape: Sequence[int], rows: Optional[Tuple[int, int]] = None,
             cols: Optional[Tuple[int, int]] = None) -> torch.Tensor:
    """Memory-map a .bin of logical `shape` and return the [rows, cols] slice as a torch tensor
    (bf16 -> torch.bfloat16, fp8 -> torch.float8_e4m3fn).  Raises on size mismatch (truncated
    or wrong-config files are an error, not a crash later)."""
    n = int(np.prod(shape))
    item = np.dtype(_NP[dtype]).itemsize
    sz = os.path.getsize(path)
    if sz != n * item:
        raise ValueError(f"{path}: expected {n * item} bytes for shape {tuple(shape)} {dtype}, found {sz}")
    mm = np.memmap(path, dtype=_NP[dtype], mode="r", shape=tuple(shape))
    if rows is not None:
        mm = mm[rows[0]:rows[1]]
    if cols is not None:
        mm = mm[..., cols[0]:cols[1]]
    t = torch.from_numpy(np.array(mm))
    if dtype == "bf16":
        t = t.view(torch.bfloat16)
    elif dtype == "fp8_e4m3":
        t = t.view(torch.float8_e4m3fn)
    return t


@dataclass
class LinearWeight:
    """A linear layer's weight in device layout ``[out, in]``.

    kind: bf16|fp16|fp32 (plain), int8|w8a8 (int8 + per-out-channel scale/zero, w = q*s+z;
    w8a8 additionally keeps the row sums for the zero-point correction), int4 / nf4 (two 4-bit
    codes per byte along `in`, low nibble first), fp8 (e4m3 + fp32 scale per 128x128 block,
    ``scale[out/128, in/128]``).  Reference staging struct: DenseLayerParams
    (src/common/llm_params.h:21-80).
    """
    kind: str
    w: torch.Tensor
    scale: Optional[torch.Tensor] = None
    zero: Optional[torch.Tensor] = None
    wsum: Optional[torch.Tensor] = None      # w8a8: sum over `in` of q, fp32 [out]
    block: int = 128
    in_features: int = 0
    out_features: int = 0
    cache: dict = field(default_factory=dict, repr=False)   # native-side descriptors

    def to(self, device) -> "LinearWeight":
        f = lambda t: None if t is None else t.to(device)
        return LinearWeight(self.kind, f(self.w), f(self.scale), f(self.zero), f(self.wsum), self.block,
                            self.in_features, self.out_features)

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w, self.scale, self.zero, self.wsum) if t is not None)


def make_linear(w_out_in: torch.Tensor, kind: str, device=None, act_dtype: torch.dtype = torch.bfloat16,
                scale: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None) -> LinearWeight:
    """Build a LinearWeight of `kind` from a dense (or pre-quantised) [out,in] tensor.

    Mirrors MMHelper::convertWeight (src/utils/matmul_helper.h:149-373): fp -> {fp16,bf16,int8,
    w8a8,uint4,nf4} quantised per output channel; int8/uint4 inputs with given scale/zero
    (GPTQ checkpoints) are kept as they are; e4m3 -> e4m3."""
    o = w_out_in.shape[0]
    if device is not None:
        w_out_in = w_out_in.to(device)
        scale = None if scale is None else scale.to(device)
        zero = None if zero is None else zero.to(device)
    if kind in ("bf16", "fp16", "fp32"):
        dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[kind]
        if w_out_in.dtype == torch.float8_e4m3fn:
            raise ValueError("fp8 weights need kind='fp8'")
        w = w_out_in.to(dt).contiguous()
        return LinearWeight(kind, w, in_features=w.shape[1], out_features=o)
    # dense weights that are already on the GPU are quantised there by one kernel per matrix (same arithmetic as the
    # PyTorch formulation in ops.reference, which serves CPU tensors)
    on_gpu = w_out_in.is_cuda and w_out_in.dtype in (torch.float32, torch.float16, torch.bfloat16)
    if kind in ("int8", "w8a8"):
        ws = None
        if w_out_in.dtype == torch.int8 and scale is not None:
            q, s, z = w_out_in.contiguous(), scale.float(), zero.float()
        elif on_gpu:
            from ..ops import native_quant
            q, s, z, ws = native_quant.quantize_rows(w_out_in, kind)
        else:
            q, s, z = R.quantize_int8_per_channel(w_out_in)
        if kind == "w8a8" and ws is None:
            ws = q.float().sum(1)
        return LinearWeight(kind, q, s, z, ws, in_features=q.shape[1], out_features=o)
    if kind == "int4":
        if w_out_in.dtype == torch.uint8 and scale is not None:
            p, s, z = w_out_in.contiguous(), scale.float(), zero.float()
        elif on_gpu and w_out_in.shape[1] % 2 == 0:
            from ..ops import native_quant
            p, s, z, _ = native_quant.quantize_rows(w_out_in, kind)
        else:
            p, s, z = R.quantize_uint4_per_channel(w_out_in)
        return LinearWeight(kind, p, s, z, in_features=p.shape[1] * 2, out_features=o)
    if kind == "nf4":
        if on_gpu and w_out_in.shape[1] % 2 == 0:
            from ..ops import native_quant
            p, s, z, _ = native_quant.quantize_rows(w_out_in, kind)
        else:
            p, s, z = R.quantize_nf4_per_channel(w_out_in)
        return LinearWeight(kind, p, s, z, in_features=p.shape[1] * 2, out_features=o)
    if kind == "fp8":
        if w_out_in.dtype == torch.float8_e4m3fn:
            if scale is None:
                raise ValueError("fp8 weight needs its block scales")
            q, s = w_out_in.contiguous(), scale.float().contiguous()
        else:
            q, s = R.quantize_fp8_block(w_out_in)
        return LinearWeight(kind, q, s, in_features=q.shape[1], out_features=o)
    raise ValueError(f"unknown weight kind {kind}")


def cat_linear(ws: Sequence[LinearWeight]) -> LinearWeight:
    """Concatenate along the out dimension (merged gate‖up, q_a‖kv_a)."""
    k = ws[0].kind
    assert all(w.kind == k for w in ws)
    cat = lambda name: None if getattr(ws[0], name) is None else torch.cat([getattr(w, name) for w in ws], 0)
    if k == "fp8":
        for w in ws[:-1]:
            assert w.out_features % w.block == 0, "fp8 concat needs 128-aligned out dims"
    return LinearWeight(k, cat("w"), cat("scale"), cat("zero"), cat("wsum"), ws[0].block, ws[0].in_features,
                        sum(w.out_features for w in ws))


class WeightSource:
    """Reads tensors of one converted model directory (or fabricates them in fake mode)."""

    def __init__(self, path: str, weight_dtype: str, device: torch.device, fake: Optional[int] = None,
                 seed: int = 0):
        self.path = path
        self.dtype = weight_dtype
        self.device = device
        self.fake = Env.get().fake_model if fake is None else fake
        self.seed = seed
        self.loaded_bytes = 0

    # -- helpers ----------------------------------------------------------------------
    def exists(self, name: str) -> bool:
        if self.fake:
            return False
        return os.path.exists(os.path.join(self.path, name))

    def _fake(self, shape, dtype: torch.dtype, name: str, std: float = 0.02, ones: bool = False) -> torch.Tensor:
        if Env.get().fake_load_info:
            print(f"[fake load] {name} {tuple(shape)}")
        if self.fake == 1:
            return torch.ones(shape, dtype=dtype, device=self.device) if ones else \
                torch.zeros(shape, dtype=dtype, device=self.device)
        if ones:
            return torch.ones(shape, dtype=dtype, device=self.device)
        g = torch.Generator(device=self.device)
        g.manual_seed((zlib.crc32(name.encode()) + self.seed) & 0x7FFFFFFF)
        t = torch.empty(shape, dtype=torch.float32 if self.device.type == "cpu" else dtype, device=self.device)
        t.normal_(0.0, std, generator=g)
        return t.to(dtype)

    def vector(self, name: str, n: int, dtype: Optional[str] = None, out_dtype=torch.float32,
               rng: Optional[Tuple[int, int]] = None, fake_ones: bool = False) -> torch.Tensor:
        """1-D tensor (norm weights, biases); optional [start,end) slice."""
        if self.fake:
            m = n if rng is None else rng[1] - rng[0]
            return self._fake((m,), out_dtype, name, ones=fake_ones)
        t = read_bin(os.path.join(self.path, name), dtype or self.dtype, (n,), rows=rng)
        self.loaded_bytes += t.numel() * t.element_size()
        return t.to(out_dtype).to(self.device)

    def matrix(self, name: str, shape: Tuple[int, int], dtype: Optional[str] = None,
               rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None) -> torch.Tensor:
        """2-D tensor in file orientation (slice applied), on the target device."""
        if self.fake:
            r = shape[0] if rows is None else rows[1] - rows[0]
            c = shape[1] if cols is None else cols[1] - cols[0]
            return self._fake((r, c), torch.bfloat16, name)
        t = read_bin(os.path.join(self.path, name), dtype or self.dtype, shape, rows=rows, cols=cols)
        self.loaded_bytes += t.numel() * t.element_size()
        return t.to(self.device)

    def linear(self, name: str, in_f: int, out_f: int, kind: str, in_rng: Optional[Tuple[int, int]] = None,
               out_rng: Optional[Tuple[int, int]] = None, out_ranges: Optional[Sequence[Tuple[int, int]]] = None,
               transposed_on_disk: bool = False, dtype: Optional[str] = None) -> LinearWeight:
        """Load ``<name>`` ([in,out] on disk unless `transposed_on_disk`) -> LinearWeight [out,in].

        `in_rng` / `out_rng` select a TP slice; `out_ranges` concatenates several out-ranges
        (q‖k‖v head ranges of the merged QKV tensor)."""
        if self.fake:
            i = in_f if in_rng is None else in_rng[1] - in_rng[0]
            if out_ranges is not None:
                o = sum(e - s for s, e in out_ranges)
            else:
                o = out_f if out_rng is None else out_rng[1] - out_rng[0]
            if kind == "fp8" and self.fake != 1:
                w = self._fake((o, i), torch.bfloat16, name)
                return make_linear(w, kind)
            return make_linear(self._fake((o, i), torch.bfloat16 if kind != "fp16" else torch.float16, name), kind)
        ranges = out_ranges if out_ranges is not None else [out_rng]
        parts = []
        fdt = dtype or self.dtype
        for rg in ranges:
            if transposed_on_disk:
                t = read_bin(os.path.join(self.path, name), fdt, (out_f, in_f), rows=rg, cols=in_rng)
            else:
                t = read_bin(os.path.join(self.path, name), fdt, (in_f, out_f), rows=in_rng, cols=rg)
            parts.append(t)
            self.loaded_bytes += t.numel() * t.element_size()
        if transposed_on_disk:
            w = torch.cat(parts, 0) if len(parts) > 1 else parts[0]
            w = w.to(self.device)
        else:
            w = torch.cat(parts, 1) if len(parts) > 1 else parts[0]
            w = w.to(self.device).t().contiguous()
        return make_linear(w, kind)

    def fp8_linear(self, name: str, in_f: int, out_f: int, in_rng=None, out_rng=None, kind: str = "fp8") -> LinearWeight:
        """DeepSeek projection: ``<name>.weight.bin`` uint8 e4m3 [in,out] (or bf16 when converted so) +
        ``<name>.weight_scale_inv.bin`` fp32 [ceil(in/128), ceil(out/128)] (format:
        deepseek_moe_convert.py:117-180; decoder_block.h:526-587).  Slices must be 128-aligned."""
        wname = name + ".weight.bin"
        if self.fake or self.dtype != "fp8_e4m3":
            return self.linear(wname, in_f, out_f, kind if self.dtype == "fp8_e4m3" or self.fake else kind,
                               in_rng, out_rng)
        B = 128
        for rg in (in_rng, out_rng):
            if rg is not None and (rg[0] % B or (rg[1] % B and rg[1] not in (in_f, out_f))):
                raise ValueError(f"fp8 slice {rg} of {name} is not 128-aligned")
        w = read_bin(os.path.join(self.path, wname), "fp8_e4m3", (in_f, out_f), rows=in_rng, cols=out_rng)
        sb = lambda rg, full: None if rg is None else (rg[0] // B, (rg[1] + B - 1) // B)
        s = read_bin(os.path.join(self.path, name + ".weight_scale_inv.bin"), "fp32",
                     ((in_f + B - 1) // B, (out_f + B - 1) // B), rows=sb(in_rng, in_f), cols=sb(out_rng, out_f))
        self.loaded_bytes += w.numel() + s.numel() * 4
        w = w.to(self.device).view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)
        s = s.to(self.device).t().contiguous()
        if kind == "fp8":
            return make_linear(w, "fp8", scale=s)
        dense = R.dequant_weight(LinearWeight("fp8", w, s, in_features=w.shape[1], out_features=w.shape[0]))
        return make_linear(dense, kind)

    def gptq_linear(self, prefix: str, in_f: int, out_f: int, qtype: str, kind: str,
                    in_rng=None, out_rng=None, out_ranges=None) -> LinearWeight:
        """GPTQ-converted tensors ``<prefix>.qweight.0.bin`` (+ ``.scales.0.bin``, ``.zeros.0.bin``):
        int8 [in,out] or uint4 packed along out, low nibble = even column
        (decoder_block.h:204-277, llama_convert.py:335-392).  The device layout packs along `in`,
        so uint4 data is unpacked, transposed and repacked here."""
        ranges = out_ranges if out_ranges is not None else [out_rng if out_rng is not None else (0, out_f)]
        qs, ss, zs = [], [], []
        for (s0, s1) in ranges:
            if qtype == "int8":
                q = read_bin(os.path.join(self.path, prefix + ".qweight.0.bin"), "int8", (in_f, out_f),
                             rows=in_rng, cols=(s0, s1))
            else:
                if s0 % 2 or s1 % 2:
                    raise ValueError("uint4 out-slices must be even")
                p = read_bin(os.path.join(self.path, prefix + ".qweight.0.bin"), "uint8", (in_f, out_f // 2),
                             rows=in_rng, cols=(s0 // 2, s1 // 2))
                q = R.unpack_nibbles(p)
            qs.append(q)
            ss.append(read_bin(os.path.join(self.path, prefix + ".scales.0.bin"), "fp32", (out_f,), rows=(s0, s1)))
            zs.append(read_bin(os.path.join(self.path, prefix + ".zeros.0.bin"), "fp32", (out_f,), rows=(s0, s1)))
        q = torch.cat(qs, 1).t().contiguous().to(self.device)
        s = torch.cat(ss).to(self.device)
        z = torch.cat(zs).to(self.device)
        if qtype == "int8" and kind in ("int8", "w8a8"):
            return make_linear(q, kind, scale=s, zero=z)
        if qtype == "uint4" and kind == "int4":
            return make_linear(R.pack_nibbles(q), kind, scale=s, zero=z)
        dense = q.float() * s[:, None] + z[:, None]
        return make_linear(dense, kind)
