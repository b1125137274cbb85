"""Group-wise low-bit quantisation for KV-cache tensors -- CUDA implementation.

Mirror of the reference's ``quantize.py`` (same names, arguments, shapes, error
types and byte format), with every tensor operation replaced by one launch of a
hand-written sm_100a kernel through the C ABI:

* ``pack_codes``            -> ``tkv_pack_codes``      (quantize.py:149-169)
* ``unpack_codes``          -> ``tkv_unpack_codes``    (quantize.py:172-183)
* ``quantize_groupwise``    -> ``tkv_quantize_pack``   (quantize.py:186-236)
* ``dequantize_groupwise``  -> ``tkv_dequantize``      (quantize.py:239-246)

Scheme: asymmetric, per group of ``group_size`` contiguous elements of the last
axis: ``scale = (max-min)/(2**nbits-1)`` (1 for a constant group), ``zero = min``,
both rounded to fp16 *before* ``code = clamp(round((x-zero)/scale))``;
``x_hat = code*scale + zero``.  Packing is split-P: with ``P = 8//nbits`` and
``DP = head_dim//P``, ``packed[..., j]`` bits ``[p*nbits, (p+1)*nbits)`` hold
``code[..., j + p*DP]``.

Tensors must live on a CUDA device; there is no CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _cabi

SUPPORTED_BITS = (2, 4)

# Metadata (scale + zero) is stored in fp16: 2 parameters x 16 bits per group.
_META_BITS_PER_GROUP = 2 * 16


def _check_bits(nbits: int) -> None:
    if nbits not in SUPPORTED_BITS:
        raise ValueError(f"nbits must be one of {SUPPORTED_BITS}, got {nbits}")


@dataclass
class QuantizedTensor:
    """A group-wise quantised tensor plus everything needed to invert it
    (the reference's container, quantize.py:73-146).

    packed: uint8 ``(*batch, head_dim // P)``; scale, zero: float16
    ``(*batch, head_dim // group_size)``.
    """

    packed: torch.Tensor
    scale: torch.Tensor
    zero: torch.Tensor
    nbits: int
    group_size: int
    head_dim: int

    @property
    def codes_per_byte(self) -> int:
        return 8 // self.nbits

    @property
    def n_groups(self) -> int:
        return self.head_dim // self.group_size

    @property
    def batch_shape(self) -> torch.Size:
        return self.packed.shape[:-1]

    @property
    def shape(self) -> torch.Size:
        return torch.Size((*self.batch_shape, self.head_dim))

    @property
    def device(self) -> torch.device:
        return self.packed.device

    def nbytes(self) -> int:
        """Actual bytes of storage, including metadata."""
        return (
            self.packed.numel() * self.packed.element_size()
            + self.scale.numel() * self.scale.element_size()
            + self.zero.numel() * self.zero.element_size()
        )

    def effective_bits_per_element(self) -> float:
        """Bits per element including the fp16 scale and zero (4-bit, group 32 -> 5.0)."""
        return self.nbits + _META_BITS_PER_GROUP / self.group_size

    def to(self, *args, **kwargs) -> "QuantizedTensor":
        return QuantizedTensor(
            packed=self.packed.to(*args, **kwargs),
            scale=self.scale.to(*args, **kwargs),
            zero=self.zero.to(*args, **kwargs),
            nbits=self.nbits,
            group_size=self.group_size,
            head_dim=self.head_dim,
        )

    def contiguous(self) -> "QuantizedTensor":
        return QuantizedTensor(
            packed=self.packed.contiguous(),
            scale=self.scale.contiguous(),
            zero=self.zero.contiguous(),
            nbits=self.nbits,
            group_size=self.group_size,
            head_dim=self.head_dim,
        )


def check_cache_tensors(qt: "QuantizedTensor", what: str, device) -> None:
    """The kernels read ``packed`` as bytes and ``scale``/``zero`` as fp16 on one device:
    anything else would be reinterpreted silently, so it is refused here.  (The reference's
    Triton loads accept any float dtype for the metadata; its quantiser only ever produces
    fp16, quantize.py:222-229.)"""
    if qt.packed.dtype != torch.uint8:
        raise TypeError(f"{what}.packed must be uint8, got {qt.packed.dtype}")
    for name in ("scale", "zero"):
        t = getattr(qt, name)
        if t.dtype != torch.float16:
            raise TypeError(f"{what}.{name} must be float16, got {t.dtype}; convert with .half()")
    for name in ("packed", "scale", "zero"):
        t = getattr(qt, name)
        if t.device != device:
            raise ValueError(f"{what}.{name} is on {t.device}, expected {device}")


def _rows(t: torch.Tensor) -> int:
    n = 1
    for s in t.shape[:-1]:
        n *= s
    return n


def pack_codes(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """Pack ``uint8`` codes ``(..., D)`` into the split-P layout ``(..., D // P)``."""
    _check_bits(nbits)
    if codes.dtype != torch.uint8:
        raise TypeError(f"codes must be uint8, got {codes.dtype}")
    P = 8 // nbits
    D = codes.shape[-1]
    if D % P != 0:
        raise ValueError(f"head_dim {D} must be divisible by {P} for {nbits}-bit packing")
    _cabi.require_cuda(codes, "codes")
    lib = _cabi.load()
    codes = codes.contiguous()
    packed = torch.empty((*codes.shape[:-1], D // P), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        _cabi.check(lib.tkv_pack_codes(codes.data_ptr(), packed.data_ptr(), _rows(codes), D, nbits,
                                       _cabi.stream_ptr(codes.device)))
    return packed


def unpack_codes(packed: torch.Tensor, nbits: int, head_dim: int) -> torch.Tensor:
    """Inverse of :func:`pack_codes`. Returns ``(..., head_dim)`` uint8."""
    _check_bits(nbits)
    P = 8 // nbits
    DP = head_dim // P
    if packed.shape[-1] != DP:
        raise ValueError(f"packed last dim {packed.shape[-1]} != head_dim//P = {DP}")
    if packed.dtype != torch.uint8:
        raise TypeError(f"packed must be uint8, got {packed.dtype}")
    _cabi.require_cuda(packed, "packed")
    lib = _cabi.load()
    packed = packed.contiguous()
    codes = torch.empty((*packed.shape[:-1], head_dim), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _cabi.check(lib.tkv_unpack_codes(packed.data_ptr(), codes.data_ptr(), _rows(packed),
                                         head_dim, nbits, _cabi.stream_ptr(packed.device)))
    return codes


def quantize_groupwise(x: torch.Tensor, nbits: int, group_size: int) -> QuantizedTensor:
    """Group-wise asymmetric quantisation along the last axis, one kernel launch.

    x: ``(..., head_dim)`` float tensor on a CUDA device; nbits 2 or 4;
    ``group_size`` must divide ``head_dim``.  Bit-exact with the reference.
    """
    _check_bits(nbits)
    D = x.shape[-1]
    if group_size <= 0 or D % group_size != 0:
        raise ValueError(f"group_size {group_size} must divide head_dim {D}")
    P = 8 // nbits
    if D % P != 0:
        raise ValueError(f"head_dim {D} must be divisible by {P} for {nbits}-bit packing")
    _cabi.require_cuda(x, "x")
    lib = _cabi.load()
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        x = x.float()  # what the reference's `.float()` does to any other dtype
    x = x.contiguous()
    batch = x.shape[:-1]
    packed = torch.empty((*batch, D // P), dtype=torch.uint8, device=x.device)
    scale = torch.empty((*batch, D // group_size), dtype=torch.float16, device=x.device)
    zero = torch.empty_like(scale)
    with torch.cuda.device(x.device):
        _cabi.check(lib.tkv_quantize_pack(x.data_ptr(), _cabi.dtype_code(x), packed.data_ptr(),
                                          scale.data_ptr(), zero.data_ptr(), _rows(x), D, nbits,
                                          group_size, _cabi.stream_ptr(x.device)))
    return QuantizedTensor(packed=packed, scale=scale, zero=zero, nbits=nbits,
                           group_size=group_size, head_dim=D)


def dequantize_groupwise(qt: QuantizedTensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of :func:`quantize_groupwise`. Returns ``(..., head_dim)`` of ``dtype``."""
    _check_bits(qt.nbits)
    _cabi.require_cuda(qt.packed, "qt.packed")
    lib = _cabi.load()
    if dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported dtype {dtype}; expected float16, bfloat16 or float32")
    check_cache_tensors(qt, "qt", qt.packed.device)
    packed, scale, zero = qt.packed.contiguous(), qt.scale.contiguous(), qt.zero.contiguous()
    out = torch.empty((*packed.shape[:-1], qt.head_dim), dtype=dtype, device=packed.device)
    code = {torch.float16: _cabi.DTYPE_F16, torch.bfloat16: _cabi.DTYPE_BF16,
            torch.float32: _cabi.DTYPE_F32}[dtype]
    with torch.cuda.device(packed.device):
        _cabi.check(lib.tkv_dequantize(packed.data_ptr(), scale.data_ptr(), zero.data_ptr(),
                                       out.data_ptr(), code, _rows(packed), qt.head_dim, qt.nbits,
                                       qt.group_size, _cabi.stream_ptr(packed.device)))
    return out


def quantize_kv(
    k: torch.Tensor, v: torch.Tensor, nbits: int, group_size: int
) -> tuple[QuantizedTensor, QuantizedTensor]:
    """Quantise a K and a V cache independently (they get their own statistics)."""
    return (
        quantize_groupwise(k, nbits, group_size).contiguous(),
        quantize_groupwise(v, nbits, group_size).contiguous(),
    )


# ---------------------------------------------------------------------------------------
# Keys quantised per channel with an fp16 residual window.  The reference describes this
# format as future work (docs/future_work.md:229-293) and does not implement it; there is
# no reference counterpart for anything below.
# ---------------------------------------------------------------------------------------

CHANNEL_GROUP_TOKENS = 32  # tokens per key group == tokens per kernel tile


@dataclass
class ChannelKeys:
    """Keys quantised per channel: a group is 32 consecutive tokens of one head dimension.

    packed: uint8 ``(B, HKV, S_q, head_dim // P)`` in the usual split-P byte layout;
    scale, zero: float16 ``(B, HKV, S_q // 32, head_dim)``."""

    packed: torch.Tensor
    scale: torch.Tensor
    zero: torch.Tensor
    nbits: int
    head_dim: int

    @property
    def tokens(self) -> int:
        return self.packed.shape[2]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.packed, self.scale, self.zero))

    def effective_bits_per_element(self) -> float:
        """Bits per element including scale and zero: the same 32 bits per 32 elements as
        per-token groups of 32 (4-bit -> 5.0)."""
        return self.nbits + _META_BITS_PER_GROUP / CHANNEL_GROUP_TOKENS


def quantize_keys_per_channel(k: torch.Tensor, nbits: int) -> tuple[ChannelKeys, torch.Tensor]:
    """k ``(B, HKV, S, D)`` -> (keys of the first ``S_q = S - S % 32`` tokens quantised per
    channel, the last ``S - S_q`` tokens as float16 ``(B, HKV, S - S_q, D)``).  A channel that
    is large for every token gets its own scale instead of flattening the small channels of
    its per-token group, which is what makes 2-bit keys usable.  One kernel launch; same
    per-element arithmetic as :func:`quantize_groupwise`, on the token axis."""
    _check_bits(nbits)
    if k.dim() != 4:
        raise ValueError(f"k must be (B, HKV, S, D), got {tuple(k.shape)}")
    B, HKV, S, D = k.shape
    P = 8 // nbits
    if D % P != 0:
        raise ValueError(f"head_dim {D} must be divisible by {P} for {nbits}-bit packing")
    _cabi.require_cuda(k, "k")
    lib = _cabi.load()
    if k.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        k = k.float()
    k = k.contiguous()
    G = CHANNEL_GROUP_TOKENS
    S_q = S - S % G
    packed = torch.empty((B, HKV, S_q, D // P), dtype=torch.uint8, device=k.device)
    scale = torch.empty((B, HKV, S_q // G, D), dtype=torch.float16, device=k.device)
    zero = torch.empty_like(scale)
    with torch.cuda.device(k.device):
        _cabi.check(lib.tkv_quantize_keys_per_channel(
            k.data_ptr(), _cabi.dtype_code(k), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(),
            B * HKV, S, S_q, D, nbits, _cabi.stream_ptr(k.device)))
    return (ChannelKeys(packed, scale, zero, nbits, D),
            k[:, :, S_q:].to(torch.float16).contiguous())


def dequantize_keys_per_channel(kc: ChannelKeys, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``code * scale + zero`` per (token block, dimension), evaluated in float32 then cast.
    A utility for tests and error reports; the decode kernel never expands the codes."""
    codes = unpack_codes(kc.packed, kc.nbits, kc.head_dim).to(torch.float32)
    B, HKV, S_q, D = codes.shape
    G = CHANNEL_GROUP_TOKENS
    cg = codes.view(B, HKV, S_q // G, G, D)
    out = cg * kc.scale.float()[:, :, :, None] + kc.zero.float()[:, :, :, None]
    return out.view(B, HKV, S_q, D).to(dtype)


def empty_cache(B: int, HKV: int, S_cap: int, head_dim: int, nbits: int, group_size: int,
                device) -> QuantizedTensor:
    """A zeroed packed cache with room for ``S_cap`` tokens per (sequence, head), to be
    filled by :func:`append_groupwise`.  No reference counterpart (the reference quantises
    whole tensors); rows past a sequence's length are never read when ``seq_lens`` is given
    to the decode functions."""
    _check_bits(nbits)
    P = 8 // nbits
    if group_size <= 0 or head_dim % group_size != 0:
        raise ValueError(f"group_size {group_size} must divide head_dim {head_dim}")
    packed = torch.zeros((B, HKV, S_cap, head_dim // P), dtype=torch.uint8, device=device)
    scale = torch.zeros((B, HKV, S_cap, head_dim // group_size), dtype=torch.float16, device=device)
    return QuantizedTensor(packed=packed, scale=scale, zero=torch.zeros_like(scale), nbits=nbits,
                           group_size=group_size, head_dim=head_dim)


def append_groupwise(cache: QuantizedTensor, x_new: torch.Tensor, positions) -> QuantizedTensor:
    """Quantise ``x_new (B, HKV, T_new, D)`` and write it in place into ``cache``
    ``(B, HKV, S_cap, ...)`` at token rows ``positions[b] + t`` (``positions``: an int for
    all sequences, or an int32 CUDA tensor ``(B,)``).  One launch, no allocation; the bytes
    written equal those of :func:`quantize_groupwise` on the same values.  Tokens that would
    land outside the cache are dropped."""
    _check_bits(cache.nbits)
    _cabi.require_cuda(x_new, "x_new")
    if x_new.dim() != 4 or cache.packed.dim() != 4:
        raise ValueError("append expects x_new (B, HKV, T_new, D) and a cache (B, HKV, S_cap, ...)")
    B, HKV, T_new, D = x_new.shape
    Bc, Hc, S_cap, _ = cache.packed.shape
    if (B, HKV, D) != (Bc, Hc, cache.head_dim):
        raise ValueError(f"x_new {tuple(x_new.shape)} does not match the cache {tuple(cache.packed.shape)}")
    if not (cache.packed.is_contiguous() and cache.scale.is_contiguous() and cache.zero.is_contiguous()):
        raise ValueError("the cache must be contiguous to be written in place")
    if x_new.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        x_new = x_new.float()
    x_new = x_new.contiguous()
    pos_ptr, pos0 = None, 0
    if isinstance(positions, torch.Tensor):
        if positions.dtype != torch.int32 or positions.shape != (B,) or positions.device != x_new.device:
            raise ValueError("positions must be an int32 tensor of shape (B,) on the cache's device")
        positions = positions.contiguous()
        pos_ptr = positions.data_ptr()
    else:
        pos0 = int(positions)
        if pos0 < 0 or pos0 + T_new > S_cap:
            raise ValueError(f"tokens [{pos0}, {pos0 + T_new}) do not fit a cache of {S_cap} rows")
    with torch.cuda.device(x_new.device):
        _cabi.check(_cabi.load().tkv_quantize_append(
            x_new.data_ptr(), _cabi.dtype_code(x_new), cache.packed.data_ptr(), cache.scale.data_ptr(),
            cache.zero.data_ptr(), B, HKV, T_new, S_cap, D, cache.nbits, cache.group_size, pos_ptr,
            pos0, _cabi.stream_ptr(x_new.device)))
    return cache


def append_kv(kq: QuantizedTensor, vq: QuantizedTensor, k_new: torch.Tensor, v_new: torch.Tensor,
              positions) -> tuple[QuantizedTensor, QuantizedTensor]:
    """Append new K and V tokens to their caches (see :func:`append_groupwise`)."""
    return append_groupwise(kq, k_new, positions), append_groupwise(vq, v_new, positions)


def roundtrip_error(x: torch.Tensor, nbits: int, group_size: int) -> dict[str, float]:
    """Quantise/dequantise ``x`` and report the reconstruction error."""
    qt = quantize_groupwise(x, nbits, group_size)
    xh = dequantize_groupwise(qt, dtype=torch.float32)
    xf = x.float()
    err = xh - xf
    denom = xf.norm().clamp_min(1e-12)
    return {
        "max_abs_err": err.abs().max().item(),
        "rel_l2": (err.norm() / denom).item(),
        "cosine": torch.nn.functional.cosine_similarity(
            xh.flatten().unsqueeze(0), xf.flatten().unsqueeze(0)
        ).item(),
        "effective_bits": qt.effective_bits_per_element(),
        "bytes": qt.nbytes(),
        "fp16_bytes": x.numel() * 2,
    }
