"""NVFP4: the 4-bit floating-point weight container, its packer, the activation-outlier metric and the linear layer.

Format (the reference's container, candle-gen/src/quant/nvfp4.rs:90-358): E2M1 codes, two per byte with the even
column in the low nibble; one unsigned E4M3 scale per block of 16 columns, stored in 128-row x 4-block atoms (the
layout block-scaled tensor-core instructions read); one fp32 scale per tensor. w = e2m1 * e4m3 * global.

The packer is bit-exact with the reference's scalar packer (nearest code, ties to the even code index) but runs as
whole-tensor torch ops. On the GPU the weights feed `swb_gemm_nvfp4` (decode-sized token counts: raw bytes stream
through TMA, 16 warps expand them to bf16 tiles in shared memory, tcgen05 multiplies) or `swb_dequant_nvfp4` followed
by the dense GEMM (prefill-sized). Activations stay bf16 (the reference's W4A16 regime); the W4A4 regime is provided as
a numerics-faithful emulation that rounds activations to the NVFP4 grid first (`quantize_activations`), not as a
native FP4 x FP4 tensor-core GEMM.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch

BLOCK = 16
E2M1_MAX = 6.0
E4M3_MAX = 448.0
SF_ATOM_ROWS = 128
SF_ATOM_COLS = 4
E2M1_MAGS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def e4m3_table() -> torch.Tensor:
    """fp32 values of the E4M3 codes 0x00..0x7E (monotonic)."""
    return torch.arange(0, 0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float()


def e4m3_from_f32(v: torch.Tensor) -> torch.Tensor:
    """Nearest non-negative E4M3 code (uint8); ties go to the even code; NaN and v <= 0 give 0."""
    tab = e4m3_table().to(v.device)
    x = torch.nan_to_num(v.float(), nan=0.0).clamp(min=0.0, max=E4M3_MAX)
    hi = torch.searchsorted(tab, x.contiguous(), right=False).clamp(max=tab.numel() - 1)
    lo = (hi - 1).clamp(min=0)
    d_lo, d_hi = (x - tab[lo]).abs(), (tab[hi] - x).abs()
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = torch.where(pick_hi, hi, lo)
    return torch.where(v > 0, code, torch.zeros_like(code)).to(torch.uint8)


def e2m1_from_f32(v: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 code (uint8, sign in bit 3); ties go to the even magnitude index; NaN gives 0."""
    v = v.float()
    mags = torch.tensor(E2M1_MAGS, dtype=torch.float32, device=v.device)
    mag = v.abs().clamp(max=E2M1_MAX)
    d = (mags - mag.unsqueeze(-1)).abs()
    dmin = d.min(dim=-1, keepdim=True).values
    cand = d == dmin
    first = cand.to(torch.uint8).argmax(dim=-1)
    nxt = (first + 1).clamp(max=7)
    tie_next = cand.gather(-1, nxt.unsqueeze(-1)).squeeze(-1) & (nxt != first)
    idx = torch.where((first % 2 == 1) & tie_next, nxt, first)
    sign = torch.signbit(v).to(torch.uint8) * 8
    code = sign | idx.to(torch.uint8)
    return torch.where(torch.isnan(v), torch.zeros_like(code), code)


def scale_offset(r: torch.Tensor | int, blk: torch.Tensor | int, sf_rows: int):
    """Byte offset of the scale of (row r, block blk) in the atom-swizzled scale tensor."""
    m_atom, k_atom = r // SF_ATOM_ROWS, blk // SF_ATOM_COLS
    atom = m_atom + (sf_rows // SF_ATOM_ROWS) * k_atom
    mr, kc = r % SF_ATOM_ROWS, blk % SF_ATOM_COLS
    return atom * (SF_ATOM_ROWS * SF_ATOM_COLS) + (mr % 32) * 16 + (mr // 32) * 4 + kc


@dataclass
class Nvfp4Tensor:
    rows: int
    cols: int
    cols_padded: int
    packed: torch.Tensor        # uint8 [rows, cols_padded / 2]
    scales: torch.Tensor        # uint8 [sf_rows * sf_cols], atom-swizzled
    sf_rows: int
    sf_cols: int
    global_scale: float

    @property
    def blocks_per_row(self) -> int:
        return self.cols_padded // BLOCK

    @staticmethod
    def scale_tensor_len(rows: int, cols: int) -> int:
        return _round_up(rows, SF_ATOM_ROWS) * _round_up(_round_up(cols, BLOCK) // BLOCK, SF_ATOM_COLS)

    @classmethod
    def pack(cls, weight: torch.Tensor) -> "Nvfp4Tensor":
        w = weight.detach().float()
        rows, cols = w.shape
        dev = w.device
        cols_padded = _round_up(cols, BLOCK)
        nb = cols_padded // BLOCK
        sf_rows, sf_cols = _round_up(rows, SF_ATOM_ROWS), _round_up(nb, SF_ATOM_COLS)
        amax = float(w.abs().max()) if w.numel() else 0.0
        f32 = torch.float32
        gs = (torch.tensor(amax, dtype=f32) / torch.tensor(E2M1_MAX * E4M3_MAX, dtype=f32)).item() if amax > 0 else 1.0
        wp = torch.zeros((rows, cols_padded), dtype=f32, device=dev)
        wp[:, :cols] = w
        blocks = wp.view(rows, nb, BLOCK)
        a_blk = blocks.abs().amax(dim=-1)
        sf_real = a_blk / torch.tensor(E2M1_MAX * gs, dtype=f32).to(dev)
        sf_byte = e4m3_from_f32(sf_real)                                    # [rows, nb]
        elem = e4m3_table().to(dev)[sf_byte.long()] * torch.tensor(gs, dtype=f32).to(dev)
        q = blocks / elem.unsqueeze(-1)
        codes = torch.where((elem > 0).unsqueeze(-1), e2m1_from_f32(q), torch.zeros_like(q, dtype=torch.uint8))
        codes = codes.view(rows, cols_padded)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
        scales = torch.zeros(sf_rows * sf_cols, dtype=torch.uint8, device=dev)
        r = torch.arange(rows, device=dev).unsqueeze(1).expand(rows, nb)
        b = torch.arange(nb, device=dev).unsqueeze(0).expand(rows, nb)
        scales[scale_offset(r, b, sf_rows).reshape(-1)] = sf_byte.reshape(-1)
        return cls(rows, cols, cols_padded, packed, scales, sf_rows, sf_cols, gs)

    def block_scales(self) -> torch.Tensor:
        """fp32 [rows, blocks_per_row]: e4m3 * global, gathered out of the swizzled layout."""
        dev = self.packed.device
        nb = self.blocks_per_row
        r = torch.arange(self.rows, device=dev).unsqueeze(1).expand(self.rows, nb)
        b = torch.arange(nb, device=dev).unsqueeze(0).expand(self.rows, nb)
        sf = self.scales[scale_offset(r, b, self.sf_rows).reshape(-1)].view(self.rows, nb)
        return e4m3_table().to(dev)[sf.long()] * torch.tensor(self.global_scale, dtype=torch.float32).to(dev)

    def dequantize(self) -> torch.Tensor:
        """fp32 [rows, cols] (the reference's `dequantize_to_vec`)."""
        dev = self.packed.device
        lut = torch.tensor(E2M1_MAGS + tuple(-m for m in E2M1_MAGS), dtype=torch.float32, device=dev)
        codes = torch.stack([self.packed & 0xF, self.packed >> 4], dim=-1).view(self.rows, self.cols_padded)
        vals = lut[codes.long()].view(self.rows, self.blocks_per_row, BLOCK) * self.block_scales().unsqueeze(-1)
        return vals.view(self.rows, self.cols_padded)[:, : self.cols].contiguous()

    def to(self, device) -> "Nvfp4Tensor":
        return Nvfp4Tensor(self.rows, self.cols, self.cols_padded, self.packed.to(device), self.scales.to(device),
                           self.sf_rows, self.sf_cols, self.global_scale)

    def nbytes(self) -> int:
        return self.packed.numel() + self.scales.numel() + 4


def quantize_device_raw(x: torch.Tensor):
    """The device packer without any host synchronisation: (codes uint8 [rows, cols / 2], scale atoms uint8, tensor
    scale as a one-element device tensor). cols must be a multiple of 16."""
    from .._native import kernels
    from .runtime import check, stream_ptr

    assert x.is_cuda and x.dim() == 2 and x.dtype in (torch.float32, torch.bfloat16) and x.stride(1) == 1
    rows, cols = x.shape
    assert cols % BLOCK == 0
    nb = cols // BLOCK
    sf_rows, sf_cols = _round_up(rows, SF_ATOM_ROWS), _round_up(nb, SF_ATOM_COLS)
    dev = x.device
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    # padding rows / columns of the scale atoms must read as zero; an exactly tiled tensor writes every byte
    alloc = torch.empty if (rows % SF_ATOM_ROWS == 0 and nb % SF_ATOM_COLS == 0) else torch.zeros
    scales = alloc(sf_rows * sf_cols, dtype=torch.uint8, device=dev)
    small = torch.zeros(2, dtype=torch.int32, device=dev)           # [tensor amax bits, tensor scale]
    gs = small[1:].view(torch.float32)
    # no per-block amax scratch: the packing kernel recomputes each block's maximum from the values it loads anyway
    check(kernels().swb_nvfp4_quantize_fast(x.data_ptr(), 1 if x.dtype == torch.float32 else 0, x.stride(0), rows, cols,
                                            packed.data_ptr(), scales.data_ptr(), sf_rows, small.data_ptr(), gs.data_ptr(),
                                            stream_ptr()), "swb_nvfp4_quantize_fast")
    return packed, scales, gs


def gemm_w4a4(x: torch.Tensor, w: "Nvfp4Tensor", bias: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] (bf16 / fp32, CUDA) times an NVFP4 weight [N, K] on the block-scaled FP4 tensor-core path: the
    activations are packed to NVFP4 by the device quantiser, then one tcgen05 kind::mxf4nvf4 GEMM produces bf16 [T, N]."""
    from .._native import kernels
    from .runtime import check, ptr, stream_ptr

    assert x.is_cuda and x.dim() == 2 and x.shape[1] == w.cols == w.cols_padded and w.cols % 256 == 0 and w.rows % 16 == 0
    aq, sfa, gs = quantize_device_raw(x.contiguous())
    T = x.shape[0]
    out = torch.empty((T, w.rows), dtype=torch.bfloat16, device=x.device)
    check(kernels().swb_gemm_nvfp4_w4a4(aq.data_ptr(), sfa.data_ptr(), gs.data_ptr(), w.packed.data_ptr(), w.scales.data_ptr(),
                                        w.global_scale, out.data_ptr(), out.stride(0), T, w.rows, w.cols, ptr(bias),
                                        stream_ptr()), "swb_gemm_nvfp4_w4a4")
    return out


def native_w4a4_enabled() -> bool:
    import os

    return os.environ.get("SWB_NVFP4_NATIVE", "1") != "0"


def quantize_on_device(x: torch.Tensor) -> Nvfp4Tensor:
    """The packer as two device kernels (block amax + tensor amax, then scales / codes / swizzle); bit-identical
    to `Nvfp4Tensor.pack`. x: CUDA fp32 or bf16 [rows, cols] with cols a multiple of 16."""
    from .._native import kernels
    from .runtime import check, stream_ptr

    assert x.is_cuda and x.dim() == 2 and x.dtype in (torch.float32, torch.bfloat16) and x.stride(1) == 1
    rows, cols = x.shape
    if cols % BLOCK != 0:
        return Nvfp4Tensor.pack(x).to(x.device)
    nb = cols // BLOCK
    sf_rows, sf_cols = _round_up(rows, SF_ATOM_ROWS), _round_up(nb, SF_ATOM_COLS)
    dev = x.device
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    scales = torch.zeros(sf_rows * sf_cols, dtype=torch.uint8, device=dev)
    block_amax = torch.empty(rows * nb, dtype=torch.float32, device=dev)
    tmax = torch.zeros(1, dtype=torch.int32, device=dev)
    gs = torch.empty(1, dtype=torch.float32, device=dev)
    check(kernels().swb_nvfp4_quantize(x.data_ptr(), 1 if x.dtype == torch.float32 else 0, x.stride(0), rows, cols,
                                       packed.data_ptr(), scales.data_ptr(), sf_rows, block_amax.data_ptr(),
                                       tmax.data_ptr(), gs.data_ptr(), stream_ptr()), "swb_nvfp4_quantize")
    return Nvfp4Tensor(rows, cols, cols, packed, scales, sf_rows, sf_cols, float(gs.item()))


def quantize_activations(x: torch.Tensor) -> torch.Tensor:
    """Rounds activations [rows, cols] to the NVFP4 grid (per-tensor scale, per-16 block scales) and returns them in
    x's dtype: what a W4A4 GEMM sees on its activation side (the reference's fused activation quantiser,
    candle-gen/src/quant/nvfp4_quant.cu:80-156, followed by the decode the tensor core performs)."""
    x2 = x.reshape(-1, x.shape[-1])
    t = quantize_on_device(x2.contiguous()) if x2.is_cuda and x2.dtype in (torch.float32, torch.bfloat16) else \
        Nvfp4Tensor.pack(x2)
    return t.dequantize().view(x.shape).to(x.dtype)


# ---- activation-outlier metric (candle-gen/src/quant/nvfp4_outlier.rs) -------------------------------------------------
class OutlierClass(enum.Enum):
    BENIGN = "benign"
    SPARSE = "sparse"
    DENSE = "dense"


@dataclass(frozen=True)
class OutlierSparsity:
    total_blocks: int
    outlier_blocks: int
    benign_fraction: float
    robust_scale: float
    max_crush_ratio: float
    tau: float

    DEFAULT_TAU = 20.0
    BENIGN_FLOOR = 0.995
    DENSE_FLOOR = 0.98

    @classmethod
    def from_tensor(cls, x: torch.Tensor, tau: float = 20.0) -> "OutlierSparsity":
        """A block of 16 is an outlier block when any magnitude exceeds tau x the median non-zero magnitude of the
        tensor; its crush ratio is max / (upper) median of the block."""
        cols = x.shape[-1] if x.dim() else 0
        data = x.detach().float().reshape(-1, cols) if cols else x.detach().float().reshape(0, 0)
        rows = data.shape[0]
        mags = data.abs().flatten()
        mags = mags[mags > 0]
        robust = float(mags.sort().values[mags.numel() // 2]) if mags.numel() else 0.0
        thr = tau * robust
        nb = (cols + BLOCK - 1) // BLOCK
        total = rows * nb
        if total == 0:
            return cls(0, 0, 1.0, robust, 0.0, tau)
        pad = nb * BLOCK - cols
        a = torch.nn.functional.pad(data.abs(), (0, pad), value=float("nan")).view(rows, nb, BLOCK)
        amax = torch.nan_to_num(a, nan=0.0).amax(-1)
        hit = (torch.nan_to_num(a, nan=0.0) > thr).any(-1) if thr > 0 else torch.zeros_like(amax, dtype=torch.bool)
        n_valid = (~torch.isnan(a)).sum(-1)
        srt = torch.nan_to_num(a, nan=float("inf")).sort(dim=-1).values       # padding sorts last
        med = srt.gather(-1, (n_valid // 2).clamp(max=BLOCK - 1).unsqueeze(-1)).squeeze(-1)
        ratio = torch.where(hit & (med > 0), amax / med, torch.zeros_like(amax))
        outliers = int(hit.sum())
        return cls(total, outliers, 1.0 - outliers / total, robust, float(ratio.max()) if outliers else 0.0, tau)

    def klass(self) -> OutlierClass:
        if self.benign_fraction >= self.BENIGN_FLOOR:
            return OutlierClass.BENIGN
        return OutlierClass.SPARSE if self.benign_fraction >= self.DENSE_FLOOR else OutlierClass.DENSE

    def w4a4_viable(self) -> bool:
        return self.klass() is not OutlierClass.DENSE


# ---- per-layer activation precision policy (candle-gen/src/quant/nvfp4_linear.rs:80-260) --------------------------------
class ActPrecision(enum.Enum):
    W4A4 = "w4a4"
    W4A16 = "w4a16"

    @staticmethod
    def _names_final_proj(l: str) -> bool:
        if "blocks." in l or "block_" in l:
            return False
        segs = l.split(".")
        tail = segs[-2] if segs[-1] in ("weight", "bias") and len(segs) > 1 else segs[-1]
        return tail == "proj_out"

    @classmethod
    def for_outlier_layer(cls, layer_name: str, is_final_proj: bool = False) -> "ActPrecision":
        """Layers whose activations carry dense outliers keep bf16 activations: caption projections, the whole
        cross-attention block, the trunk's final projection, the first and last transformer blocks."""
        l = layer_name.lower()
        outlier = ("caption_projection" in l or "caption_proj" in l or "attn2" in l or "cross_att" in l
                   or "crossatt" in l
                   or ("cross" in l and any(t in l for t in ("_k", "_v", ".k", ".v")))
                   or is_final_proj or cls._names_final_proj(l)
                   or "blocks.0." in l or "block_0." in l or "last_block" in l or "final_block" in l)
        return cls.W4A16 if outlier else cls.W4A4


@dataclass
class Nvfp4Partition:
    assignments: list[tuple[str, ActPrecision]]
    n_w4a4: int
    n_w4a16: int

    @classmethod
    def of(cls, names) -> "Nvfp4Partition":
        a = [(n, ActPrecision.for_outlier_layer(n)) for n in names]
        n4 = sum(1 for _, p in a if p is ActPrecision.W4A4)
        return cls(a, n4, len(a) - n4)

    def w4a4_fraction(self) -> float:
        t = self.n_w4a4 + self.n_w4a16
        return self.n_w4a4 / t if t else 0.0


# ---- linear layer -------------------------------------------------------------------------------------------------------
class Nvfp4Linear:
    """y = x W^T + b with W stored as NVFP4 (candle-gen/src/quant/nvfp4_linear.rs:463-800).

    On a CUDA device with `act_precision=W4A4` and more than 64 token rows, activations are packed to NVFP4 on the
    device and the product runs on the block-scaled FP4 tensor-core kernel (`gemm_w4a4`). Otherwise: up to 64 token rows run the fused dequantise-and-multiply kernel; more rows expand the weight
    to bf16 once per call (or once for good with `keep_dense=True`) and run the dense tcgen05 GEMM. On the CPU the
    dequantised weight is multiplied in fp32 (the oracle). `act_precision=W4A4` rounds activations to the NVFP4
    grid before the multiply."""

    def __init__(self, tensor: Nvfp4Tensor, bias: torch.Tensor | None = None,
                 act_precision: ActPrecision = ActPrecision.W4A16, keep_dense: bool = False):
        if tensor.cols % 256 != 0 and tensor.packed.is_cuda:
            raise ValueError("the NVFP4 kernels need the input dimension to be a multiple of 256")
        self.t, self.bias, self.act_precision, self.keep_dense = tensor, bias, act_precision, keep_dense
        self._dense: torch.Tensor | None = None

    @classmethod
    def from_dense(cls, weight: torch.Tensor, bias: torch.Tensor | None = None, layer_name: str | None = None,
                   **kw) -> "Nvfp4Linear":
        if layer_name is not None:
            kw.setdefault("act_precision", ActPrecision.for_outlier_layer(layer_name))
        dev = weight.device
        return cls(Nvfp4Tensor.pack(weight).to(dev), bias, **kw)

    @property
    def shape(self) -> tuple[int, int]:
        return self.t.rows, self.t.cols

    def nvfp4_footprint_bytes(self) -> int:
        return self.t.nbytes()

    def bf16_footprint_bytes(self) -> int:
        return self.t.rows * self.t.cols * 2

    def dense_bf16(self) -> torch.Tensor:
        t = self.t
        if not t.packed.is_cuda:
            return t.dequantize().to(torch.bfloat16)
        if self._dense is not None:
            return self._dense
        from .._native import kernels
        from .runtime import check, stream_ptr

        out = torch.empty((t.rows, t.cols), dtype=torch.bfloat16, device=t.packed.device)
        check(kernels().swb_dequant_nvfp4(t.packed.data_ptr(), t.scales.data_ptr(), t.global_scale, out.data_ptr(),
                                          t.rows, t.cols, stream_ptr()), "swb_dequant_nvfp4")
        if self.keep_dense:
            self._dense = out
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        t = self.t
        if (self.act_precision is ActPrecision.W4A4 and t.packed.is_cuda and x2.shape[0] > 64 and t.rows % 16 == 0 and
                x2.dtype in (torch.float32, torch.bfloat16) and native_w4a4_enabled()):
            # both operands stay 4-bit all the way into the tensor core
            return gemm_w4a4(x2, t, self.bias).to(x.dtype).reshape(*lead, t.rows)
        if self.act_precision is ActPrecision.W4A4:
            x2 = quantize_activations(x2)
        if not t.packed.is_cuda:
            y = x2.float() @ t.dequantize().t()
            if self.bias is not None:
                y = y + self.bias.float()
            return y.to(x.dtype).reshape(*lead, t.rows)
        from .._native import kernels
        from .gemm import gemm_bf16, gemm_workspace
        from .runtime import check, ptr, stream_ptr

        x2 = x2.to(torch.bfloat16).contiguous()
        T = x2.shape[0]
        if T <= 64 and self._dense is None:
            out = torch.empty((T, t.rows), dtype=torch.bfloat16, device=x2.device)
            ws = gemm_workspace(x2.device)
            check(kernels().swb_gemm_nvfp4(x2.data_ptr(), x2.stride(0), t.packed.data_ptr(), t.scales.data_ptr(),
                                           t.global_scale, out.data_ptr(), out.stride(0), T, t.rows, t.cols,
                                           ptr(self.bias), ws.data_ptr(), ws.numel(), 0, stream_ptr()),
                  "swb_gemm_nvfp4")
        else:
            out = gemm_bf16(x2, self.dense_bf16(), bias=self.bias)
        return out.reshape(*lead, t.rows)

    __call__ = forward
