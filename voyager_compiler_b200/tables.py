"""Host-side construction and analysis of the 65 536-entry bf16 lookup tables (``qmap``).

voyager-compiler describes every element format by a table that maps each bf16 bit pattern to a
representable value (``get_quantization_map``, src/voyager_compiler/quantization/
fake_quantize.py:30-98).  When this package is used as a drop-in, the upstream code builds the
tables and merely passes them to the ops; the builders below exist so the kernels can be used,
tested and benchmarked stand-alone.  They are written against integer bit patterns with numpy
and are checked bit for bit against tables produced by the upstream builders.

The second half analyses a table so the kernels can replace the gather by something cheaper
when that is provably the same function:

* ``INT``  - the table equals ``clamp(round_half_even(v), lo, hi)``;
* ``RUNS`` - the table is piecewise constant over the ordered finite bf16 numbers with at most 512
  runs: a sorted array of run starts and a branchless binary search in shared memory;
* ``LUT16`` - anything else: the full table, staged in shared memory.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

__all__ = [
    "bf16_patterns_f32", "f32_to_bf16_bits", "bf16_bits_to_f32", "build_table", "codebook_table",
    "quant_range", "TableAnalysis", "analyse_table", "sort_key", "code_table",
]

_ALL = np.arange(1 << 16, dtype=np.uint32)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns; every NaN becomes 0x7FC0 | sign."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32)
    nan = np.isnan(x)
    r = np.where(nan, 0x7FC0 | ((u >> 16) & 0x8000).astype(np.uint32), r)
    return r.astype(np.uint16)


def bf16_patterns_f32() -> np.ndarray:
    """fp32 value of every bf16 pattern, in pattern order."""
    return bf16_bits_to_f32(_ALL)


def _r(x):
    """Round an fp32/fp64 array to bf16 and return it as fp32 (one bf16 arithmetic step)."""
    with np.errstate(all="ignore"):
        return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))


def _true_exponent(v: np.ndarray) -> np.ndarray:
    """floor(log2 |v|) for finite non-zero v, from the bits (bf16 subnormals included)."""
    m, e = np.frexp(np.abs(v).astype(np.float64))
    return (e - 1).astype(np.int64)


# ---------------------------------------------------------------------------------------------
# builders
# ---------------------------------------------------------------------------------------------
def _int_table(lo: float, hi: float) -> np.ndarray:
    v = bf16_patterns_f32()
    with np.errstate(all="ignore"):
        return f32_to_bf16_bits(np.clip(np.rint(v), lo, hi))


def _minifloat_table(mbits: int, vmax: float, emin: int) -> np.ndarray:
    """Saturating fp8-style grid with subnormals (``e4m3`` / ``e5m2`` strings)."""
    with np.errstate(all="ignore"):
        v = bf16_patterns_f32().astype(np.float64)
    a = np.abs(v)
    fin = np.isfinite(v)
    nz = fin & (a > 0)
    e = np.zeros(v.shape, dtype=np.int64)
    e[nz] = _true_exponent(v[nz])
    step = np.exp2((np.maximum(e, emin) - mbits).astype(np.float64))
    with np.errstate(all="ignore"):
        q = np.rint(a / step) * step
    q = np.minimum(q, vmax) * np.sign(v)
    q = np.where(nz & (q != 0), q, 0.0)            # every zero result is +0
    q = np.where(fin, q, np.nan)
    return f32_to_bf16_bits(q.astype(np.float32))


def _posit_table(nbits: int, es: int) -> np.ndarray:
    """Posit(nbits, es): round to nearest on the posit bit string, ties to the even string."""
    with np.errstate(all="ignore"):
        v = bf16_patterns_f32().astype(np.float64)
    out = np.zeros(v.shape, dtype=np.float64)
    useed_log = 1 << es
    smax = (nbits - 2) * useed_log
    cut = 2.0 ** math.floor(-(nbits - 1) * useed_log + 2 ** (es - 1))
    F = 23  # fraction bits carried (bf16 has 7; 23 keeps the arithmetic generic)
    for i in range(1 << 16):
        x = v[i]
        if not np.isfinite(x):
            out[i] = np.nan
            continue
        a = abs(x)
        if a == 0 or a < cut:
            out[i] = 0.0
            continue
        m, e2 = math.frexp(a)
        sc = e2 - 1
        frac = int(round((m * 2 - 1) * (1 << F)))
        if sc > smax:
            out[i] = math.copysign(2.0 ** smax, x)
            continue
        if sc < -smax:
            out[i] = math.copysign(2.0 ** -smax, x)
            continue
        k, ex = sc >> es, sc & (useed_log - 1)
        if k >= 0:
            regime, rlen = ((1 << (k + 1)) - 1) << 1, k + 2
        else:
            regime, rlen = 1, -k + 1
        body = (((regime << es) | ex) << F) | frac
        total = rlen + es + F
        drop = total - (nbits - 1)
        if drop > 0:
            keep, rest = body >> drop, body & ((1 << drop) - 1)
            half = 1 << (drop - 1)
            if rest > half or (rest == half and (keep & 1)):
                keep += 1
        else:
            keep = body << (-drop)
        keep = min(keep, (1 << (nbits - 1)) - 1)
        out[i] = math.copysign(_posit_decode(keep, nbits, es), x)
    return f32_to_bf16_bits(out.astype(np.float32))


def _posit_decode(p: int, nbits: int, es: int) -> float:
    """Value of a positive posit bit string ``p`` (nbits-1 bits, sign stripped)."""
    if p == 0:
        return 0.0
    width = nbits - 1
    bits = [(p >> (width - 1 - j)) & 1 for j in range(width)]
    first = bits[0]
    run = 1
    while run < width and bits[run] == first:
        run += 1
    k = run - 1 if first else -run
    pos = run + 1  # skip the terminating bit
    ex = 0
    for j in range(es):
        ex <<= 1
        if pos < width:
            ex |= bits[pos]
        pos += 1
    frac, scale = 0.0, 0.5
    while pos < width:
        frac += bits[pos] * scale
        scale /= 2
        pos += 1
    return (2.0 ** (k * (1 << es) + ex)) * (1.0 + frac)


def _scaled_float_table(n: int, ebits: int, mbits: int, name: str) -> np.ndarray:
    """``fpN_eXmY`` strings: the microscaling element rule evaluated step by step in bf16
    arithmetic, which is what gives these tables their non-monotone corners."""
    x = bf16_patterns_f32()
    if n == ebits + mbits:          # unsigned variant used for scale factors
        x = np.abs(x)
    bits = mbits + 2
    emax = 2 ** (ebits - 1) - 1 if ebits > 4 else 2 ** (ebits - 1)
    max_norm = 2 ** emax * 1.75 if name == "fp8_e4m3" else 2 ** emax * float(2 ** (bits - 1) - 1) / 2 ** (bits - 2)
    with np.errstate(all="ignore"):
        mag = _r(np.abs(x) + (x == 0).astype(np.float32))
        pe = np.floor(_r(np.log2(mag.astype(np.float64))))
        pe = np.maximum(pe, -(2 ** (ebits - 1)) + 2).astype(np.float32)
        p2 = _r(np.exp2(pe.astype(np.float64)))
        up = np.float32(2.0 ** (bits - 2))
        out = _r(_r(x / p2) * up)
        a = np.abs(out)
        tie = (np.mod(_r(a - 0.5), 2) == 0).astype(np.float32)
        out = _r(np.sign(out) * _r(np.floor(_r(a + 0.5)) - tie))
        out = _r(_r(out / up) * p2)
        out = np.clip(out, -max_norm, max_norm)     # NaN stays NaN
        out = np.where(x == np.inf, np.inf, out)
        out = np.where(x == -np.inf, -np.inf, out)
    return f32_to_bf16_bits(out.astype(np.float32))


def nf_levels(k: int = 4, int_bits: Optional[int] = None) -> np.ndarray:
    """NormalFloat levels (QLoRA construction, asymmetric: 2^(k-1) positive, 2^(k-1)-1 negative
    quantiles of N(0,1) plus zero, normalised to max 1), as bf16-rounded fp32."""
    import torch  # linspace must be torch's fp32 linspace to reproduce the upstream levels
    from scipy.stats import norm

    half = 2 ** (k - 1)
    offset = 0.9677083
    pos = norm.ppf(torch.linspace(offset, 0.5, half + 1)[:-1].numpy()).tolist()
    neg = (-norm.ppf(torch.linspace(offset, 0.5, half)[:-1].numpy())).tolist()
    lv = np.sort(np.asarray(pos + [0.0] + neg, dtype=np.float32))
    lv = lv / lv.max()
    if int_bits is not None:
        lv = np.rint(lv * np.float32(2 ** (int_bits - 1) - 1)).astype(np.float32)
    return _r(lv)


def _nf_table(k: int, int_bits: Optional[int]) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    lv = nf_levels(k, int_bits)
    x = bf16_patterns_f32()
    with np.errstate(all="ignore"):
        xc = np.clip(x, lv.min(), lv.max())
        d = np.abs(_r(lv[None, :] - xc[:, None]))
    idx = np.where(np.isnan(x), 0, np.argmin(np.where(np.isnan(d), np.inf, d), axis=1))
    return f32_to_bf16_bits(lv[idx]), idx.astype(np.uint8), lv


def codebook_table(entries: Sequence[float]) -> np.ndarray:
    """Nearest entry of an arbitrary codebook in fp32, ties to the lower index, NaN to entry 0."""
    cb = np.asarray(list(entries), dtype=np.float32)
    x = bf16_patterns_f32()
    with np.errstate(all="ignore"):
        d = np.abs(np.clip(x, cb.min(), cb.max())[:, None] - cb[None, :])
    idx = np.where(np.isnan(x), 0, np.argmin(np.where(np.isnan(d), np.inf, d), axis=1))
    return f32_to_bf16_bits(cb[idx])


def build_table(dtype: Optional[str]) -> np.ndarray:
    """uint16[65536]: bf16 bit pattern of the value each bf16 pattern quantizes to.

    Accepts the upstream dtype strings: ``intN``, ``uintN``, ``e4m3``/``e5m2`` (optionally
    ``fp8.`` prefixed), ``fpN_eXmY``, ``positN_E``, ``nfK`` / ``nfK_B``, ``float32`` /
    ``bfloat16`` / ``float16`` and ``None`` (identity)."""
    if dtype is None or dtype in ("float32", "bfloat16"):
        t = _ALL.astype(np.uint16)
        return t
    if dtype == "float16":
        with np.errstate(all="ignore"):
            return f32_to_bf16_bits(bf16_patterns_f32().astype(np.float16).astype(np.float32))
    if m := re.fullmatch(r"int(\d+)", dtype, re.IGNORECASE):
        n = int(m.group(1))
        return _int_table(-(2 ** (n - 1)), 2 ** (n - 1) - 1)
    if m := re.fullmatch(r"uint(\d+)", dtype, re.IGNORECASE):
        return _int_table(0, 2 ** int(m.group(1)) - 1)
    if m := re.fullmatch(r"(?:fp8\.)?(e4m3|e5m2)", dtype, re.IGNORECASE):
        return _minifloat_table(3, 448.0, -6) if m.group(1).lower() == "e4m3" else _minifloat_table(2, 57344.0, -14)
    if m := re.fullmatch(r"fp(\d+)_e(\d+)m(\d+)", dtype):
        n, eb, mb = map(int, m.groups())
        if n not in (eb + mb, eb + mb + 1):
            raise ValueError(f"inconsistent float format: {dtype}")
        return _scaled_float_table(n, eb, mb, dtype)
    if m := re.fullmatch(r"posit(\d+)_(\d+)", dtype):
        return _posit_table(int(m.group(1)), int(m.group(2)))
    if m := re.fullmatch(r"nf(\d+)(?:_(\d+))?", dtype):
        return _nf_table(int(m.group(1)), int(m.group(2)) if m.group(2) else None)[0]
    raise ValueError(f"Unsupported dtype: {dtype}")


def quant_range(dtype: str) -> Tuple[float, float]:
    """(quant_min, quant_max) of a format string, with the upstream conventions
    (src/voyager_compiler/quantization/qspec.py:65-105): posit -> maxpos, nfK -> 1, nfK_B -> 2^(B-1)-1."""
    if m := re.fullmatch(r"int(\d+)", dtype, re.IGNORECASE):
        n = int(m.group(1))
        return float(-(2 ** (n - 1))), float(2 ** (n - 1) - 1)
    if m := re.fullmatch(r"uint(\d+)", dtype, re.IGNORECASE):
        return 0.0, float(2 ** int(m.group(1)) - 1)
    if m := re.fullmatch(r"(?:fp8\.)?(e4m3|e5m2)", dtype, re.IGNORECASE):
        hi = 448.0 if m.group(1).lower() == "e4m3" else 57344.0
        return -hi, hi
    if m := re.fullmatch(r"fp(\d+)_e(\d+)m(\d+)", dtype, re.IGNORECASE):
        eb, mb = int(m.group(2)), int(m.group(3)) + 2
        emax = 2 ** (eb - 1) - 1 if eb > 4 else 2 ** (eb - 1)
        hi = 2 ** emax * 1.75 if dtype.lower() == "fp8_e4m3" else 2 ** emax * (2 ** (mb - 1) - 1) / 2 ** (mb - 2)
        return -float(hi), float(hi)
    if m := re.fullmatch(r"posit(\d+)_(\d+)", dtype, re.IGNORECASE):
        hi = float((2 ** (2 ** int(m.group(2)))) ** (int(m.group(1)) - 2))
        return -hi, hi
    if m := re.fullmatch(r"nf(\d+)(?:_(\d+))?", dtype, re.IGNORECASE):
        hi = float(2 ** (int(m.group(2)) - 1) - 1) if m.group(2) is not None else 1.0
        return -hi, hi
    raise ValueError(f"Unsupported dtype: {dtype}")


# ---------------------------------------------------------------------------------------------
# analysis
# ---------------------------------------------------------------------------------------------
def sort_key(bits: np.ndarray) -> np.ndarray:
    """Order-preserving key of bf16 patterns: ascending key == ascending value (-0 below +0)."""
    b = bits.astype(np.uint32)
    return np.where(b & 0x8000, b ^ 0xFFFF, b ^ 0x8000).astype(np.uint32)


_IS_NAN_PATTERN = (_ALL & 0x7FFF) > 0x7F80
_IS_SPECIAL = (_ALL & 0x7F80) == 0x7F80                        # inf and NaN inputs
_ORDER = np.argsort(sort_key(_ALL)[~_IS_SPECIAL], kind="stable")
_ORDERED_PATTERNS = _ALL[~_IS_SPECIAL][_ORDER]                 # most negative finite ... most positive
_ORDERED_KEYS = sort_key(_ORDERED_PATTERNS)
MAX_RUNS = 512


def _canon(bits: np.ndarray) -> np.ndarray:
    """Collapse every NaN output pattern to one value so NaN == NaN when comparing tables."""
    b = bits.astype(np.uint32)
    return np.where((b & 0x7FFF) > 0x7F80, 0x7FC0, b).astype(np.uint16)


@dataclass
class TableAnalysis:
    lut16: np.ndarray                 # uint16[65536]
    is_int: bool
    lo: float
    hi: float
    n_runs: int                       # runs over the finite inputs; 0 when more than MAX_RUNS
    run_keys: Optional[np.ndarray]    # uint16[n_runs-1]
    run_vals: Optional[np.ndarray]    # uint16[n_runs]
    run_first: Optional[np.ndarray]   # uint32[n_runs]: a bf16 pattern inside each run
    nan_val: int                      # output pattern for NaN inputs (entry 0xFFFF)
    pinf_val: int                     # output pattern for +inf (entry 0x7F80)
    ninf_val: int                     # output pattern for -inf (entry 0xFF80)
    nan_consistent: bool              # every NaN input pattern maps to the same output
    flat_tiny: bool = False           # constant over patterns 0..0x400 and over 0x8000..0x8400


def analyse_table(lut16: np.ndarray) -> TableAnalysis:
    lut16 = np.ascontiguousarray(lut16, dtype=np.uint16)
    assert lut16.shape == (1 << 16,)
    canon = _canon(lut16)
    vals = bf16_bits_to_f32(lut16)
    nan_out = canon[_IS_NAN_PATTERN]
    nan_consistent = bool((nan_out == nan_out[0]).all())
    nan_val = int(lut16[0xFFFF])

    # INT: equal to clamp(rint(v), lo, hi) with integer bounds that are exact in bf16
    is_int, lo, hi = False, 0.0, 0.0
    fin = vals[np.isfinite(vals)]
    if fin.size:
        lo, hi = float(fin.min()), float(fin.max())
        if lo == math.floor(lo) and hi == math.floor(hi) and -256 <= lo <= hi <= 256:
            ref = _canon(_int_table(lo, hi))
            # the kernel maps a NaN input to NaN; -0 results compare by bits
            is_int = bool((ref == canon).all())

    ordered = canon[_ORDERED_PATTERNS]
    change = np.flatnonzero(ordered[1:] != ordered[:-1]) + 1
    n_runs = int(change.size + 1)
    run_keys = run_vals = run_first = None
    if n_runs <= MAX_RUNS:
        run_keys = _ORDERED_KEYS[change].astype(np.uint16)
        run_first = _ORDERED_PATTERNS[np.concatenate([[0], change])]
        run_vals = lut16[run_first].astype(np.uint16)
    else:
        n_runs = 0
    return TableAnalysis(lut16, is_int, lo, hi, n_runs, run_keys, run_vals, run_first, nan_val, int(lut16[0x7F80]),
                         int(lut16[0xFF80]), nan_consistent,
                         bool((canon[:0x401] == canon[0]).all() and (canon[0x8000:0x8401] == canon[0x8000]).all()))


def code_table(lut16: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Packed-code view of a value table: ``(lut8 uint8[65536], levels fp32[n])``.

    * every value an integer in [0, 255] (an index table): code = value, levels = 0..max;
    * every value an integer in [-128, 127]: code = two's-complement byte, levels = value of
      each byte 0..255;
    * otherwise, at most 256 distinct values: code = rank among the ascending distinct values,
      levels = those values.  NaN outputs get code = number of levels (or 0 when that is 256).
    Raises ValueError when the table has more than 256 distinct non-NaN values."""
    vals = bf16_bits_to_f32(np.ascontiguousarray(lut16, dtype=np.uint16))
    nan = np.isnan(vals)
    fin = vals[~nan]
    integral = np.isfinite(fin).all() and (fin == np.rint(fin)).all()
    if integral and fin.min() >= 0 and fin.max() <= 255:
        levels = np.arange(int(fin.max()) + 1, dtype=np.float32)
        codes = np.where(nan, 0, vals).astype(np.int64)
    elif integral and fin.min() >= -128 and fin.max() <= 127:
        levels = np.arange(256, dtype=np.int64)
        levels = np.where(levels >= 128, levels - 256, levels).astype(np.float32)
        codes = np.where(nan, 0, vals).astype(np.int64) & 0xFF
    else:
        levels = np.unique(fin.astype(np.float32))
        if levels.size > 256:
            raise ValueError(f"table has {levels.size} distinct values; packed codes need <= 256")
        codes = np.searchsorted(levels, np.where(nan, levels[0], vals)).astype(np.int64)
        codes = np.where(nan, levels.size if levels.size < 256 else 0, codes)
    return codes.astype(np.uint8), levels


def levels_by_code_and_sign(lut16: np.ndarray, codes: np.ndarray) -> Optional[np.ndarray]:
    """fp32[512]: the table's output for packed code ``c`` and an input without / with the sign bit
    at ``[c]`` / ``[256 + c]``, when the output is a function of (code, input sign) alone -- i.e.
    ``lut16[p] == out[codes[p] + 256 * (p >> 15)]`` for every pattern ``p`` (signed zeros and NaN
    payloads compared by bits).  ``None`` when it is not (e.g. 256 levels plus a NaN output that had to
    share a code)."""
    lut16 = np.ascontiguousarray(lut16, dtype=np.uint16)
    idx = codes.astype(np.int64) + 256 * (np.arange(1 << 16) >> 15)
    out = np.zeros(512, dtype=np.uint16)
    out[idx] = lut16                      # any representative; checked below
    if not np.array_equal(out[idx], lut16):
        return None
    return bf16_bits_to_f32(out).astype(np.float32)
