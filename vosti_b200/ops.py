"""Python face of the CUDA kernels: one function per kernel, taking torch tensors
that live on the GPU and launching on torch's current stream.

There is no CPU fallback and no library stand-in: if the compiled library is
missing it is built, and if that fails, or the device is not sm_100, the call
raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

_LIB = None


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The compiled kernel library, built at the first call."""
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(str(_build.library_path()))
        lib.vosti_last_error.restype = ctypes.c_char_p
        _LIB = lib
    return _LIB


_CHECKED_DEVICES = set()


def require_device(device: torch.device) -> None:
    """Fail loudly unless `device` is a CUDA device of compute capability 10.x."""
    if device.type != "cuda":
        raise KernelError(f"vosti_b200 kernels run on a CUDA device, got '{device}'")
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index in _CHECKED_DEVICES:
        return
    major, minor = torch.cuda.get_device_capability(index)
    if major != 10:
        raise KernelError(f"vosti_b200 kernels are built for sm_100a; device {index} is sm_{major}{minor}")
    _CHECKED_DEVICES.add(index)


LAUNCHES = 0   # kernels of this library launched so far (counted per launcher call)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if code != 0:
        raise KernelError(f"{what}: {library().vosti_last_error().decode()} (code {code})")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _is_f32(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _same_dtype(*tensors: torch.Tensor) -> int:
    flag = _is_f32(tensors[0])
    for t in tensors[1:]:
        if t is not None and _is_f32(t) != flag:
            raise KernelError("activation tensors of one call must share a dtype")
    return flag


def _contig(*tensors):
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor,
              feedback: Optional[tuple] = None, scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
              rounded: bool = False):
    """table[ids] * scale. `feedback` = (source, values), int32: row t takes values[source[t]] as
    its id where source[t] >= 0 (a token sampled on the device that the host has not read yet).
    `out_dtype` float32 gives float32 rows from a bfloat16 table (the scaled entry is not rounded
    again): the start of a float32 residual stream; with `rounded` the call returns a `StreamPair` of
    those rows and their rounding to bfloat16, written by the same kernel."""
    _contig(ids, table)
    source, values = feedback if feedback is not None else (None, None)
    if source is not None:
        _contig(source, values)
        assert source.shape[0] == ids.shape[0] and source.dtype == values.dtype == torch.int32
    if out_dtype == torch.float32 and table.dtype != torch.float32:
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
        low = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.bfloat16, device=table.device) if rounded else None
        _check(library().vosti_embedding_stream(_p(ids), _p(source), _p(values), _p(table), _p(out), _p(low), ids.shape[0],
                                                table.shape[1], table.shape[0], _is_f32(table), ctypes.c_float(scale), _p(status),
                                                _stream()), "embedding")
        return StreamPair(low, out) if rounded else out
    if out_dtype is not None and out_dtype != table.dtype:
        raise KernelError("embedding: rows come in the table's type or in float32")
    out = torch.empty((ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    _check(library().vosti_embedding(_p(ids), _p(source), _p(values), _p(table), _p(out), ids.shape[0], table.shape[1],
                                     table.shape[0], _is_f32(table), ctypes.c_float(scale), _p(status), _stream()),
           "embedding")
    return out


RMSNORM_PARTIAL_MAX_WIDTH = 24576    # floats of shared memory the split-summing norm keeps a row in


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            residual: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None):
    """out = rmsnorm(x [+ residual]) * weight; with `residual` the sum is written to
    `residual_out` (which may be `residual` itself). Returns (out, residual_out)."""
    if isinstance(x, PartialSum) and x.width > RMSNORM_PARTIAL_MAX_WIDTH:
        x = x.materialize()          # wider than the fused kernel's row buffer: sum the splits first
    if isinstance(x, PartialSum):
        x.check()
        _contig(weight, residual, residual_out)
        like = residual if residual is not None else None
        out = torch.empty((x.rows, x.width), dtype=x.dtype, device=x.partial.device)
        flag = _is_f32(out)
        if like is not None and _is_f32(like) != flag:
            raise KernelError("activation tensors of one call must share a dtype")
        _check(library().vosti_rmsnorm_partial(_p(x.partial), x.splits, _p(residual), _p(weight), _is_f32(weight),
                                               _p(out), _p(residual_out), x.rows, x.width, ctypes.c_float(eps), flag,
                                               _stream()), "rmsnorm_partial")
        return out, residual_out
    _contig(x, weight, residual, residual_out)
    flag = _same_dtype(x, residual, residual_out)
    out = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(library().vosti_rmsnorm(_p(x), _p(residual), _p(weight), _is_f32(weight), _p(out),
                                   _p(residual_out), rows, x.shape[-1], ctypes.c_float(eps), flag,
                                   _stream()), "rmsnorm")
    return out, residual_out


def affine_rows(x: torch.Tensor, *, bias: Optional[torch.Tensor] = None, scale: float = 1.0, softcap: float = 0.0,
                out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """cap(x * scale + bias) per row from a float32 product, rounded once to `out_dtype`:
    cap(y) = softcap * tanh(y / softcap) when softcap > 0. A float32 result overwrites x."""
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("affine_rows takes a float32 [rows, width] matrix with unit inner stride")
    _contig(bias)
    if bias is not None and bias.numel() != x.shape[1]:
        raise KernelError(f"affine_rows: bias has {bias.numel()} entries, the rows have {x.shape[1]}")
    out = x if out_dtype == torch.float32 else torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _check(library().vosti_affine_rows(_p(x), ctypes.c_int64(x.stride(0)), _p(bias),
                                       0 if bias is None else _is_f32(bias), _p(out), ctypes.c_int64(out.stride(0)),
                                       _is_f32(out), x.shape[0], x.shape[1], ctypes.c_float(scale),
                                       ctypes.c_float(softcap), _stream()), "affine_rows")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    _contig(gate_up)
    inter = gate_up.shape[-1] // 2
    out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(library().vosti_silu_mul(_p(gate_up), _p(out), gate_up.shape[0], inter, _is_f32(gate_up),
                                    _stream()), "silu_mul")
    return out


GLU_ACTIVATIONS = {"silu": 0, "relu": 1, "relu2": 2}
FUSED_GLU_ACTIVATIONS = {"silu": 2, "relu": 4, "relu2": 5}         # the tensor-core product's gated epilogues


def glu_mul(gate_up: torch.Tensor, activation: str) -> torch.Tensor:
    """act(gate) * up of a [rows, 2 * inter] product with the gate half first; `activation` is
    "silu", "relu" or "relu2" (the square of relu)."""
    if activation == "silu":
        return silu_mul(gate_up)
    _contig(gate_up)
    inter = gate_up.shape[-1] // 2
    out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(library().vosti_glu_mul(_p(gate_up), _p(out), gate_up.shape[0], inter, GLU_ACTIVATIONS[activation], _is_f32(gate_up),
                                   _stream()), "glu_mul")
    return out


def gemm_simt(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor, *,
              out_dtype: Optional[torch.dtype] = None,
              row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x[row_index] @ w.T with float32 arithmetic on the CUDA cores."""
    _contig(x, w, row_index)
    rows = x.shape[0] if row_index is None else row_index.shape[0]
    out = torch.empty((rows, w.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
    if x.shape[1] != w.shape[1]:
        raise KernelError(f"gemm: inner sizes differ ({x.shape[1]} vs {w.shape[1]})")
    _check(library().vosti_gemm_simt(_p(x), _p(w), _p(out), _p(row_index), rows, x.shape[0], w.shape[0],
                                     x.shape[1], _is_f32(x), _is_f32(w), _is_f32(out), _p(status),
                                     _stream()), "gemm_simt")
    return out


def qkv_post(qkv: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *,
             nq: int, nkv: int, head_dim: int, page_size: int = 1, q_norm_w: Optional[torch.Tensor] = None,
             k_norm_w: Optional[torch.Tensor] = None, eps: float = 1.0, cos: Optional[torch.Tensor] = None,
             sin: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
             slot_mapping: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
             rotary_dim: Optional[int] = None, interleaved: bool = False) -> torch.Tensor:
    """Head norm, rotation and cache store after the QKV projection; returns q [T, nq*d].
    `qkv` may be the projection or the unsummed partial sums of its split-K product. The
    rotation takes the first `rotary_dim` elements of a head (default: all of it) in pairs
    (i, i + rotary_dim/2), or (2i, 2i + 1) with `interleaved`; cos/sin are [positions, rotary_dim/2]."""
    partial, splits = None, 0
    if isinstance(qkv, PartialSum):
        qkv.check()
        partial, splits = qkv.partial, qkv.splits
        proxy = torch.empty((0,), dtype=qkv.dtype, device=partial.device)
        tokens, width, dtype, device = qkv.rows, qkv.width, qkv.dtype, partial.device
        qkv = None
    else:
        proxy = qkv
        tokens, width, dtype, device = qkv.shape[0], qkv.shape[1], qkv.dtype, qkv.device
    _contig(qkv, k_cache, v_cache, q_norm_w, k_norm_w, cos, sin, positions, slot_mapping)
    if width != (nq + 2 * nkv) * head_dim:
        raise KernelError("qkv_post: input width does not match the head counts")
    flag = _same_dtype(proxy, k_cache, v_cache)
    q_out = torch.empty((tokens, nq * head_dim), dtype=dtype, device=device)
    num_slots = 0 if k_cache is None else k_cache.numel() // (nkv * head_dim)
    norm_flag = 0
    if q_norm_w is not None:
        norm_flag = _is_f32(q_norm_w)
        if k_norm_w is not None and _is_f32(k_norm_w) != norm_flag:
            raise KernelError("qkv_post: q and k norm weights must share a dtype")
    elif k_norm_w is not None:
        norm_flag = _is_f32(k_norm_w)
    max_positions = 0 if cos is None else cos.shape[0]
    rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape):
        raise KernelError("qkv_post: rotation tables must be float32 [positions, rotary_dim/2]")
    _check(library().vosti_qkv_post(
        _p(qkv), _p(partial), splits, _p(q_out), _p(k_cache), _p(v_cache), _p(q_norm_w), _p(k_norm_w), norm_flag,
        ctypes.c_float(eps), _p(cos), _p(sin), max_positions, _p(positions), _p(slot_mapping),
        ctypes.c_int64(num_slots), page_size, tokens, nq, nkv, head_dim, rotary_dim, int(bool(interleaved)), flag,
        _p(status), _stream()), "qkv_post")
    return q_out


def attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, positions: torch.Tensor,
                   request_of: torch.Tensor, block_table: torch.Tensor, page_size: int, nq: int, nkv: int,
                   head_dim: int, scale: float, window: int, status: torch.Tensor) -> torch.Tensor:
    _contig(q, k_cache, v_cache, positions, request_of, block_table)
    flag = _same_dtype(q, k_cache, v_cache)
    tokens = q.shape[0]
    out = torch.empty_like(q)
    num_pages = k_cache.numel() // (page_size * nkv * head_dim)
    _check(library().vosti_attention_simt(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(positions), _p(request_of), _p(block_table),
        block_table.shape[1], page_size, num_pages, tokens, nq, nkv, head_dim, ctypes.c_float(scale),
        window, flag, _p(status), _stream()), "attention")
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tokens (int32[rows]) from float32 logits [rows, vocab], written to `out` if given."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with unit inner stride")
    _contig(temperature, seeds, counters)
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    elif out.dtype != torch.int32 or out.numel() < logits.shape[0] or not out.is_contiguous():
        raise KernelError("sample: out must be a contiguous int32 tensor with a slot per row")
    _check(library().vosti_sample(_p(logits), logits.shape[0], logits.shape[1],
                                  ctypes.c_int64(logits.stride(0)), _p(temperature), _p(seeds),
                                  _p(counters), _p(out), _stream()), "sample")
    return out


def sample_slots(logits: torch.Tensor, slots: torch.Tensor, table: torch.Tensor, positions: Optional[torch.Tensor],
                 status: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tokens from float32 logits with each row's sampler state read from, and advanced in, its
    per-request slot: `slots` int32[rows], `table` int64[slots, 4] = (temperature as float bits,
    seed, index of the next token, position)."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with unit inner stride")
    _contig(slots, table, positions)
    if slots.dtype != torch.int32 or slots.numel() < logits.shape[0] or table.dtype != torch.int64 or table.shape[-1] != 4:
        raise KernelError("sample_slots: slots must be int32 with an entry per row, the table int64 [slots, 4]")
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    elif out.dtype != torch.int32 or out.numel() < logits.shape[0] or not out.is_contiguous():
        raise KernelError("sample: out must be a contiguous int32 tensor with a slot per row")
    _check(library().vosti_sample_slots(_p(logits), logits.shape[0], logits.shape[1], ctypes.c_int64(logits.stride(0)),
                                        _p(slots), _p(table), table.shape[0], _p(positions), _p(out), _p(status),
                                        _stream()), "sample_slots")
    return out


def gemm_tc_supported(n: int, k: int) -> bool:
    """Whether the tensor-core product takes a [n, k] bfloat16 weight."""
    return bool(library().vosti_gemm_tc_supported(int(n), int(k)))


_WORKSPACES = {}
WORKSPACE_GENERATION = 0   # bumped whenever a scratch buffer moves (captured graphs hold its address)


def _workspace(device: torch.device, elems: int, purpose: str = "attention") -> torch.Tensor:
    """float32 scratch, one per device and purpose, grown on demand. Kernels on one stream
    use it one after the other."""
    key = (device.type, device.index, purpose)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < elems:
        global WORKSPACE_GENERATION
        WORKSPACE_GENERATION += 1
        buf = torch.empty(max(elems, 1 << 22), dtype=torch.float32, device=device)
        _WORKSPACES[key] = buf
    return buf


_COUNTERS = {}


def _counters(device: torch.device, count: int) -> torch.Tensor:
    """Zeroed int32 counters that kernels leave zeroed (arrival counts of the decode
    attention), one buffer per device, grown on demand."""
    key = (device.type, device.index)
    buf = _COUNTERS.get(key)
    if buf is None or buf.numel() < count:
        global WORKSPACE_GENERATION
        WORKSPACE_GENERATION += 1
        buf = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _COUNTERS[key] = buf
    return buf


EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2
_SPLIT_GENERATION = 0   # counts split-K products: a PartialSum is valid until the next one runs


class PartialSum:
    """The result of a split-K product whose splits have not been summed yet: float32
    [splits, rows, width] in the split-K scratch. A consumer that can add the splits itself
    (the fused add + RMSNorm, the head norm / rotation kernel) takes it as it is; anything else
    calls `materialize`. It must be consumed before the next split-K product runs."""

    def __init__(self, partial: torch.Tensor, splits: int, rows: int, width: int, dtype: torch.dtype,
                 status: torch.Tensor):
        self.partial, self.splits, self.rows, self.width, self.dtype = partial, splits, rows, width, dtype
        self.status = status
        self.generation = _SPLIT_GENERATION

    @property
    def shape(self):
        return (self.rows, self.width)

    def check(self) -> None:
        if self.generation != _SPLIT_GENERATION:
            raise KernelError("a deferred split-K result was used after a later split-K product overwrote it")

    def materialize(self) -> torch.Tensor:
        self.check()
        out = torch.empty((self.rows, self.width), dtype=self.dtype, device=self.partial.device)
        _check(library().vosti_splitk_reduce(_p(self.partial), _p(out), self.splits, self.rows, self.width,
                                             _is_f32(out), _stream()), "splitk_reduce")
        return out


def materialize(x):
    return x.materialize() if isinstance(x, (PartialSum, StreamPair)) else x


class PackedWeight:
    """A [features, k] bfloat16 weight stored tile by tile for the tensor-core product:
    [k blocks of 64][feature tiles of 128][128][64], zero-padded to whole tiles, so that every
    tile a CTA streams is one contiguous 16 KiB piece of memory instead of 128 row pieces of
    128 bytes."""

    TILE_F, TILE_K = 128, 64

    def __init__(self, w: torch.Tensor):
        if w.dtype != torch.bfloat16 or w.dim() != 2:
            raise KernelError("PackedWeight takes a 2-d bfloat16 matrix")
        features, k = w.shape
        ft, kb = -(-features // self.TILE_F), -(-k // self.TILE_K)
        padded = w
        if features != ft * self.TILE_F or k != kb * self.TILE_K:
            padded = torch.zeros((ft * self.TILE_F, kb * self.TILE_K), dtype=w.dtype, device=w.device)
            padded[:features, :k] = w
        self.data = padded.view(ft, self.TILE_F, kb, self.TILE_K).permute(2, 0, 1, 3).contiguous()
        self.shape = (features, k)
        self.dtype, self.device = w.dtype, w.device

    @property
    def is_cuda(self) -> bool:
        return self.data.is_cuda

    def numel(self) -> int:
        return self.data.numel()

    def element_size(self) -> int:
        return self.data.element_size()


def gemm_tc(x: torch.Tensor, w, status: torch.Tensor, *, out_dtype: Optional[torch.dtype] = None,
            swiglu: bool = False, allow_partial: bool = False, activation: str = "silu"):
    """y = x @ w.T on the tensor cores (bfloat16 operands, float32 accumulation); w is a
    [features, k] tensor or a `PackedWeight`. With `swiglu` the rows of w are blocks of 16 gate
    rows followed by their 16 up rows and y = act(gate) * up has half as many columns, act being
    `activation`: "silu", "relu" or "relu2" (the square of relu)."""
    packed = isinstance(w, PackedWeight)
    w_data = w.data if packed else w
    _contig(x, w_data)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    tokens, k = x.shape
    features = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm: inner sizes differ ({k} vs {w.shape[1]})")
    out_dtype = out_dtype or torch.bfloat16
    if swiglu:
        if activation not in FUSED_GLU_ACTIVATIONS:
            raise KernelError(f"gemm_tc: the gated epilogue takes {sorted(FUSED_GLU_ACTIVATIONS)}, not '{activation}'")
        epilogue, width = FUSED_GLU_ACTIVATIONS[activation], features // 2
        if out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the fused SiLU*up epilogue writes bfloat16")
    else:
        epilogue, width = (EPI_F32 if out_dtype == torch.float32 else EPI_BF16), features
    global _SPLIT_GENERATION
    lib = library()
    splits = lib.vosti_gemm_tc_splits(tokens, features, k)
    elems = splits * tokens * features if splits > 1 else 0
    ws = _workspace(x.device, elems, "split_k") if elems else None
    defer = bool(allow_partial and splits > 1 and epilogue in (EPI_BF16, EPI_F32))
    out = None if defer else torch.empty((tokens, width), dtype=out_dtype, device=x.device)
    if splits > 1:
        _SPLIT_GENERATION += 1
    _check(lib.vosti_gemm_tc(_p(x), _p(w_data), _p(out), tokens, features, k, epilogue, _p(ws),
                             ctypes.c_int64(ws.numel() if ws is not None else 0), int(defer), int(packed), _p(status),
                             _stream()),
           "gemm_tc", kernels=2 if splits > 1 and not defer else 1)
    if defer:
        return PartialSum(ws, splits, tokens, features, out_dtype, status)
    return out


# Weights requested ahead (see csrc/common.cuh, VostiPrefetch): the norm before a product asks for
# the start of the product's weights. VOSTI_PREFETCH=0 switches it off. Measured at the 8B sizes,
# context 2,048: 3.65 instead of 3.76 ms per step at batch 8 with 32 MB per hint (8 MB: 3.71,
# 96 MB: 3.90, slower than none). Also measured and not kept: asking for the output
# projection's weights from the head kernel or from the tail of the decode attention (the step
# got 2 % slower: the requests delay the attention's own loads by more than the projection
# gains), and asking, per K split, for the k-blocks after those the product's CTAs request by
# themselves (3.71 ms).
import os as _os
PREFETCH = _os.environ.get("VOSTI_PREFETCH", "1") != "0"
PREFETCH_LIMIT = int(_os.environ.get("VOSTI_PREFETCH_MB", "32")) << 20    # bytes asked for at most per hint
PREFETCH_MAX_TOKENS = 64         # steps with more tokens keep HBM busy anyway


def hint_prefetch(w, limit: Optional[int] = None) -> bool:
    """Name the weight the next product will stream, for the next kernel that can ask for its
    first `limit` bytes to be brought into L2 while it runs (the split-summing norm). Only
    tile-packed weights are taken (their first bytes are the first k-blocks of every feature
    tile). `None` clears a hint nobody took. Returns whether a hint was set."""
    lib = library()
    if w is None or not PREFETCH or not isinstance(w, PackedWeight):
        lib.vosti_hint_prefetch(None, ctypes.c_longlong(0))
        return False
    nbytes = min(w.data.numel() * w.data.element_size(), limit if limit is not None else PREFETCH_LIMIT)
    _check(lib.vosti_hint_prefetch(_p(w.data), ctypes.c_longlong(nbytes)), "hint_prefetch", kernels=0)
    return True


def gather_rows(x: torch.Tensor, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """x[rows] for int32 row indices (the embedding kernel over an activation matrix)."""
    return embedding(rows, x, status)


FIXED_ORDER = False              # set_fixed_order: one order of arithmetic however the work is cut


def set_fixed_order(enabled: bool) -> None:
    """Make a token's bfloat16 values the same bits however the work is cut into steps and
    batches, for this process: products never split their K range, no kernel is chosen by the
    number of tokens in the launch, and every token's attention runs on the portion kernel
    (whose rows are independent of one another and whose key tiles start at key 0). Decoding
    is slower for it: fewer CTAs stream the weights, and a lone token fills one row of a tile."""
    global FIXED_ORDER
    library().vosti_set_fixed_order(1 if enabled else 0)
    FIXED_ORDER = bool(enabled)


BATCH_INVARIANT_SEGMENT = 576    # keys per decode-attention segment when the length is pinned


def set_decode_once(enabled: bool) -> None:
    """The decode attention's kernel with one CTA per item (a cluster of CTAs per token and kv head) on or off
    for every later launch of this process; off, every launch takes the persistent kernel."""
    _check(library().vosti_set_decode_once(1 if enabled else 0), "set_decode_once", kernels=0)


def set_decode_segment(keys: int) -> None:
    """Pin the decode attention's segment length for this process (0: every launch chooses by
    its shape). Pinned, a token's attention does not depend on the size of its batch or on its
    companions' lengths, at some cost in speed for large batches."""
    _check(library().vosti_set_decode_segment(int(keys)), "set_decode_segment", kernels=0)


INVARIANCE = "off"          # the mode set last


def set_invariance(mode) -> str:
    """Choose what a token's bfloat16 bits may depend on, for the launches that follow (the
    kernel library keeps the mode; an engine sets its own mode again before each of its steps,
    so engines of one process may differ).
    False, None, "off": every launch picks the fastest cut for its shape.
    "decode": the decode attention's segment length is pinned, so a decode step of up to 64
    rows gives a row the same bits whatever the batch around it is; prompts cut differently
    agree up to rounding only.
    True, "full": one order of arithmetic everywhere (set_fixed_order): the same bits however
    the tokens are cut into steps and whatever else is in the batch."""
    name = {False: "off", None: "off", True: "full", "0": "off", "1": "full", "": "off"}.get(mode, mode)
    if name not in ("off", "decode", "full"):
        raise ValueError(f"batch invariance is 'off', 'decode' or 'full', not {mode!r}")
    global INVARIANCE
    if name != INVARIANCE:
        set_fixed_order(name == "full")
        set_decode_segment(BATCH_INVARIANT_SEGMENT if name == "decode" else 0)
        INVARIANCE = name
    return name


def attention_decode(q, k_cache, v_cache, out, *, token_list, count, positions, request_of, block_table,
                     page_size, nq, nkv, head_dim, max_kv_len, scale, window, status) -> None:
    """Single-query attention with split keys for `count` tokens (bfloat16)."""
    lib = library()
    tokens_total = q.shape[0]
    lib.vosti_attention_decode_scratch.restype = ctypes.c_int64
    elems = lib.vosti_attention_decode_scratch(count, nq, nkv, head_dim, max_kv_len)
    scratch = _workspace(q.device, elems)
    arrivals = _counters(q.device, count * nkv)
    num_pages = k_cache.numel() // (page_size * nkv * head_dim)
    _check(lib.vosti_attention_decode(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scratch), ctypes.c_int64(scratch.numel()), _p(arrivals),
        _p(token_list),
        count, tokens_total, _p(positions), _p(request_of), _p(block_table), block_table.shape[1], page_size,
        num_pages, nq, nkv, head_dim, max_kv_len, ctypes.c_float(scale), window, _p(status), _stream()),
        "attention_decode")


DECODE_FUSION = _os.environ.get("VOSTI_DECODE_FUSION", "1") != "0"


def attention_decode_fused(qkv: "PartialSum", k_cache, v_cache, *, positions, request_of, block_table, slot_mapping,
                           page_size, nq, nkv, head_dim, max_kv_len, scale, window, q_norm_w, k_norm_w, eps, cos, sin,
                           status) -> torch.Tensor:
    """Head norm, rotation, cache store and single-query attention in one kernel, for a step in
    which every request brings one token: `qkv` is the QKV projection's unsummed split-K result
    (row i = token i = request i). Returns the attention output [tokens, nq * head_dim]."""
    qkv.check()
    lib = library()
    count = qkv.rows
    if qkv.width != (nq + 2 * nkv) * head_dim or qkv.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused: the projection does not match the head counts or is not bfloat16")
    _contig(k_cache, v_cache, positions, request_of, block_table, slot_mapping, q_norm_w, k_norm_w, cos, sin)
    if block_table.dim() != 2 or block_table.shape[0] < count:
        raise KernelError("attention_decode_fused: the block table needs a row per request (one token each)")
    norm_flag = 0
    if q_norm_w is not None:
        norm_flag = _is_f32(q_norm_w)
        if k_norm_w is not None and _is_f32(k_norm_w) != norm_flag:
            raise KernelError("attention_decode_fused: q and k norm weights must share a dtype")
    elif k_norm_w is not None:
        norm_flag = _is_f32(k_norm_w)
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2):
        raise KernelError("attention_decode_fused: rotation tables must be float32 [positions, head_dim/2]")
    out = torch.empty((count, nq * head_dim), dtype=torch.bfloat16, device=qkv.partial.device)
    lib.vosti_attention_decode_scratch.restype = ctypes.c_int64
    elems = lib.vosti_attention_decode_scratch(count, nq, nkv, head_dim, max_kv_len)
    scratch = _workspace(out.device, elems)
    arrivals = _counters(out.device, count * nkv)
    num_pages = k_cache.numel() // (page_size * nkv * head_dim)
    _check(lib.vosti_attention_decode_fused(
        _p(qkv.partial), qkv.splits, _p(k_cache), _p(v_cache), _p(out), _p(scratch), ctypes.c_int64(scratch.numel()),
        _p(arrivals), count, _p(positions), _p(request_of), _p(block_table), block_table.shape[1], page_size, num_pages,
        nq, nkv, head_dim, max_kv_len, ctypes.c_float(scale), window, _p(q_norm_w), _p(k_norm_w), norm_flag,
        ctypes.c_float(eps), _p(cos), _p(sin), 0 if cos is None else cos.shape[0], _p(slot_mapping), _p(status),
        _stream()), "attention_decode_fused")
    return out


def attention_prefill(q, k_cache, v_cache, out, *, row_list, count, cu_q, kv_len, block_table, page_size, nq, nkv,
                      head_dim, max_q_len, scale, window, status, kernel: Optional[str] = None) -> None:
    """Attention of whole portions for `count` requests (bfloat16). Head sizes 64 and 128 with
    pages of a multiple of 16 tokens run on the tcgen05 kernel ("tc"), everything else on the
    mma.sync kernel ("mma"); `kernel` forces one."""
    lib = library()
    num_pages = k_cache.numel() // (page_size * nkv * head_dim)
    if kernel is None:
        kernel = "tc" if lib.vosti_attention_prefill_tc_supported(head_dim, page_size) and nq // nkv <= 16 else "mma"
    if kernel == "tc":
        _check(lib.vosti_attention_prefill_tc(
            _p(q), _p(k_cache), _p(v_cache), _p(out), _p(row_list), count, _p(cu_q), _p(kv_len), _p(block_table),
            block_table.shape[1], page_size, num_pages, nq, nkv, head_dim, max_q_len, q.shape[0],
            ctypes.c_float(scale), window, _p(status), _stream()), "attention_prefill_tc")
        return
    _check(lib.vosti_attention_prefill(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(row_list), count, _p(cu_q), _p(kv_len), _p(block_table),
        block_table.shape[1], page_size, num_pages, nq, nkv, head_dim, max_q_len, ctypes.c_float(scale), window,
        _p(status), _stream()), "attention_prefill")


SHORT_ROW = 4     # requests that bring at most this many tokens are served one query at a time


def attention_step_layout(q_lens):
    """How the attention kernels divide a step (registered with the step layout as "attention"):
    the tokens of requests that bring at most SHORT_ROW tokens go to the split-key kernel one
    query at a time, the requests that bring more to the portion kernel; with one order of
    arithmetic asked for (set_fixed_order) everything goes to the portion kernel. Lists that
    would name every token or every request are left out."""
    B = len(q_lens)
    short_tokens, long_rows, cursor = [], [], 0
    if FIXED_ORDER:
        long_rows = list(range(B))
    elif sum(q_lens) == B:
        short_tokens = list(range(B))
    else:
        for i, n in enumerate(q_lens):
            if n <= SHORT_ROW:
                short_tokens.extend(range(cursor, cursor + n))
            else:
                long_rows.append(i)
            cursor += n
    arrays = {"short_tokens": short_tokens, "long_rows": long_rows} if short_tokens and long_rows else {}
    return arrays, {"num_short_tokens": len(short_tokens), "num_long_rows": len(long_rows),
                    "max_long_q_len": max((q_lens[i] for i in long_rows), default=0)}


def attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, *, nq: int, nkv: int,
              head_dim: int, scale: float, window: int) -> torch.Tensor:
    """Attention of every query row of the batch over its request's cached keys. float32
    runs on the CUDA cores; bfloat16 on the tensor cores, requests that bring a few tokens
    one query at a time with split keys, longer portions tile by tile (the step's work lists:
    attention_step_layout)."""
    if q.dtype != torch.bfloat16 or nq // nkv > 16:
        return attention_simt(q, k_cache, v_cache, positions=ctx.positions, request_of=ctx.request_of,
                              block_table=group.block_table, page_size=group.page_size, nq=nq, nkv=nkv,
                              head_dim=head_dim, scale=scale, window=window, status=ctx.status)
    _contig(q, k_cache, v_cache)
    out = torch.empty_like(q)
    common = dict(block_table=group.block_table, page_size=group.page_size, nq=nq, nkv=nkv, head_dim=head_dim,
                  scale=scale, window=window, status=ctx.status)
    lists = ctx.layout["attention"]
    if lists["num_short_tokens"]:
        attention_decode(q, k_cache, v_cache, out, token_list=ctx.extras.get("attention.short_tokens"),
                         count=lists["num_short_tokens"], positions=ctx.positions, request_of=ctx.request_of,
                         max_kv_len=ctx.max_kv_len, **common)
    if lists["num_long_rows"]:
        attention_prefill(q, k_cache, v_cache, out, row_list=ctx.extras.get("attention.long_rows"),
                          count=lists["num_long_rows"], cu_q=ctx.cu_q, kv_len=ctx.kv_len,
                          max_q_len=lists["max_long_q_len"], **common)
    return out


# ---------------------------------------------------------------- float32 residual stream
class DeferredSum:
    """Sublayer outputs [rows, width] that still have to be added to the residual stream: the
    kernel that next reads the stream (a norm with `forward_add`, `stream_sum`) adds them in
    order, in float32. `materialize` gives their sum alone."""

    def __init__(self, *terms):
        self.terms = tuple(materialize(t) for t in terms if t is not None)
        if not 1 <= len(self.terms) <= 2:
            raise KernelError("a deferred sum holds one or two terms")
        self.shape = tuple(self.terms[0].shape)

    def materialize(self) -> torch.Tensor:
        return stream_sum(None, self)


def _terms(x):
    """Up to two addends as (pointer, is_f32) pairs."""
    if x is None:
        terms = ()
    elif isinstance(x, DeferredSum):
        terms = x.terms
    else:
        terms = (materialize(x),)
    _contig(*terms)
    flat = []
    for t in terms:
        flat += [_p(t), _is_f32(t)]
    while len(flat) < 4:
        flat += [None, 0]
    return terms, flat


def dyt(x, weight: torch.Tensor, bias: Optional[torch.Tensor], alpha: float, out_dtype: torch.dtype,
        stream: Optional[torch.Tensor] = None, stream_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dynamic Tanh of s = stream + x (x: a tensor, a `DeferredSum` or None; stream: float32 or None):
    tanh(alpha * s) * weight + bias in float32, rounded to `out_dtype`; s itself goes to
    `stream_out` (float32, may be `stream`)."""
    terms, flat = _terms(x)
    like = stream if stream is not None else terms[0]
    _contig(stream, stream_out, weight, bias)
    if stream is not None and stream.dtype != torch.float32 or stream_out is not None and stream_out.dtype != torch.float32:
        raise KernelError("dyt: the residual stream is float32")
    if bias is not None and bias.dtype != weight.dtype:
        raise KernelError("dyt: weight and bias must share a dtype")
    rows, width = like.shape
    out = torch.empty((rows, width), dtype=out_dtype, device=like.device)
    _check(library().vosti_dyt(_p(stream), *flat, _p(stream_out), _p(weight), _p(bias), _is_f32(weight),
                               ctypes.c_float(alpha), _p(out), _is_f32(out), rows, width, _stream()), "dyt")
    return out


def stream_sum(stream: Optional[torch.Tensor], x, *, out_dtype: torch.dtype = torch.float32,
               tail: Optional[torch.Tensor] = None) -> torch.Tensor:
    """stream + x in float32, rounded to `out_dtype`; with `tail` [rows, w] the result is
    [rows, width + w] with the tail's rows appended to the sum's (the operand of a product with
    a [.., width + w] weight)."""
    terms, flat = _terms(x)
    like = stream if stream is not None else terms[0]
    _contig(stream, tail)
    rows, width = like.shape
    tail_width = 0 if tail is None else tail.shape[1]
    out = torch.empty((rows, width + tail_width), dtype=out_dtype, device=like.device)
    _check(library().vosti_stream_sum(_p(stream), *flat, _p(out), _is_f32(out), ctypes.c_int64(width + tail_width),
                                      _p(tail), 0 if tail is None else _is_f32(tail), tail_width, rows, width,
                                      _stream()), "stream_sum")
    return out


def branch_merge(xs, weights, eps: float) -> torch.Tensor:
    """mean over branches of x_b / sqrt(mean(x_b^2) + eps) * w_b, float32 [rows, width]."""
    xs = [materialize(x) for x in xs]
    _contig(*xs, *weights)
    count = len(xs)
    rows, width = xs[0].shape
    flag = _is_f32(weights[0])
    if any(_is_f32(w) != flag for w in weights) or any(tuple(x.shape) != (rows, width) for x in xs):
        raise KernelError("branch_merge: branches must share a shape and their weights a dtype")
    out = torch.empty((rows, width), dtype=torch.float32, device=xs[0].device)
    x_ptrs = (ctypes.c_void_p * count)(*[x.data_ptr() for x in xs])
    w_ptrs = (ctypes.c_void_p * count)(*[w.data_ptr() for w in weights])
    kinds = (ctypes.c_int * count)(*[_is_f32(x) for x in xs])
    _check(library().vosti_branch_merge(x_ptrs, kinds, w_ptrs, flag, count, _p(out), rows, width, ctypes.c_float(eps),
                                        _stream()), "branch_merge")
    return out


def branch_sum(xs, scales) -> torch.Tensor:
    """sum over branches of scales[b] * x_b, float32 [rows, width], added in branch order."""
    xs = [materialize(x) for x in xs]
    _contig(*xs)
    count = len(xs)
    rows, width = xs[0].shape
    if len(scales) != count or any(tuple(x.shape) != (rows, width) for x in xs):
        raise KernelError("branch_sum: branches must share a shape and have a constant each")
    out = torch.empty((rows, width), dtype=torch.float32, device=xs[0].device)
    x_ptrs = (ctypes.c_void_p * count)(*[x.data_ptr() for x in xs])
    kinds = (ctypes.c_int * count)(*[_is_f32(x) for x in xs])
    consts = (ctypes.c_float * count)(*[float(c) for c in scales])
    _check(library().vosti_branch_sum(x_ptrs, kinds, consts, count, _p(out), rows, width, _stream()), "branch_sum")
    return out


def rms_stream(x, weight: Optional[torch.Tensor], eps: float, out_dtype: Optional[torch.dtype], *, offset: float = 0.0,
               stream: Optional[torch.Tensor] = None, stream_out: Optional[torch.Tensor] = None):
    """Root-mean-square norm of s = stream + x over a float32 residual stream (x: a tensor, a
    `DeferredSum` or None; stream: float32 or None): s / sqrt(mean(s^2) + eps) * (offset + weight) in
    float32, rounded to `out_dtype`; s itself goes to `stream_out` (float32, may be `stream`).
    Without a weight the result is s rounded to `out_dtype`; without `out_dtype` only the sum is
    stored and None is returned."""
    terms, flat = _terms(x)
    like = stream if stream is not None else terms[0]
    _contig(stream, stream_out, weight)
    if stream is not None and stream.dtype != torch.float32 or stream_out is not None and stream_out.dtype != torch.float32:
        raise KernelError("rms_stream: the residual stream is float32")
    rows, width = like.shape
    out = None if out_dtype is None else torch.empty((rows, width), dtype=out_dtype, device=like.device)
    _check(library().vosti_rms_stream(_p(stream), *flat, _p(stream_out), _p(weight), 0 if weight is None else _is_f32(weight),
                                      ctypes.c_float(offset), ctypes.c_float(eps), _p(out),
                                      0 if out is None else _is_f32(out), rows, width, _stream()), "rms_stream")
    return out


# ---------------------------------------------------------------- token inputs
class StreamPair:
    """A float32 residual stream [rows, width] together with its rounding to the serving type: what a
    block that norms after the sum hands to the next one (the sublayers' products read `rounded`,
    the next sum reads `stream`). In float32 serving both are one tensor. `materialize` gives the stream."""

    def __init__(self, rounded: torch.Tensor, stream: torch.Tensor):
        self.rounded, self.stream = rounded, stream
        self.shape = tuple(stream.shape)

    def materialize(self) -> torch.Tensor:
        return self.stream


def post_norm_stream(stream: torch.Tensor, x, weight: torch.Tensor, alpha: float, eps: float, out_dtype: torch.dtype, *,
                     offset: float = 0.0, in_place: bool = True) -> "StreamPair":
    """Norm after the sum: s = alpha * stream + x in float32 (x: a tensor or a `DeferredSum`),
    y = s / sqrt(mean(s^2) + eps) * (offset + weight). y becomes the stream (float32, written over the
    old one with `in_place`) and, rounded to `out_dtype`, the next sublayer's input. x may be a float32
    product's unsummed K splits (`PartialSum`), which the kernel adds in split order."""
    splits = 1
    if isinstance(x, PartialSum) and x.dtype == torch.float32:
        x.check()
        splits, x = x.splits, x.partial[: x.splits * x.rows * x.width].view(x.splits * x.rows, x.width)[: x.rows]
    terms, flat = _terms(x)
    _contig(stream, weight)
    if stream.dtype != torch.float32:
        raise KernelError("post_norm_stream: the residual stream is float32")
    rows, width = stream.shape
    if any(tuple(t.shape) != (rows, width) for t in terms) or weight.shape[0] != width:
        raise KernelError("post_norm_stream: the terms and the weight must match the stream's shape")
    new = stream if in_place else torch.empty_like(stream)
    out = None if out_dtype == torch.float32 else torch.empty((rows, width), dtype=out_dtype, device=stream.device)
    _check(library().vosti_post_norm_stream(_p(stream), ctypes.c_float(alpha), *flat, _p(weight), _is_f32(weight),
                                            ctypes.c_float(offset), ctypes.c_float(eps), _p(new), _p(out), 0, rows, width,
                                            splits, _stream()), "post_norm_stream")
    return StreamPair(new if out is None else out, new)


def pair_embedding(ids: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, last_token: torch.Tensor, ctx, *,
                   buckets: int, mul_prev: int, mul_cur: int, feedback: Optional[tuple] = None):
    """table[id] + pairs[(prev * mul_prev + id * mul_cur) % buckets] in float32, row `buckets` of
    `pairs` for tokens at position 0; `prev` is the token before in the step, or, for the first
    token of a request's portion, what `last_token` (int32 [slots]) holds for its slot, which is
    then set to the portion's last token. Returns (rows float32 [tokens, hidden], the token ids
    int32 [tokens] with those a sampler left on the device filled in)."""
    _contig(ids, table, pairs, last_token)
    source, values = feedback if feedback is not None else (None, None)
    if source is not None:
        _contig(source, values)
    if _is_f32(table) != _is_f32(pairs) or last_token.dtype != torch.int32 or pairs.shape[0] != buckets + 1:
        raise KernelError("pair_embedding: the tables must share a type, the pair table has buckets + 1 rows")
    tokens = ids.shape[0]
    out = torch.empty((tokens, table.shape[1]), dtype=torch.float32, device=table.device)
    resolved = torch.empty((tokens,), dtype=torch.int32, device=table.device)
    _check(library().vosti_pair_embedding(
        _p(ids), _p(source), _p(values), _p(ctx.positions), _p(ctx.request_of), _p(ctx.cu_q), _p(ctx.state_slots),
        _p(last_token), last_token.shape[0], ctx.num_requests, _p(table), _p(pairs), _is_f32(table), _p(out), _p(resolved),
        tokens, table.shape[1], table.shape[0], ctypes.c_longlong(buckets), ctypes.c_longlong(mul_prev),
        ctypes.c_longlong(mul_cur), _p(ctx.status), _stream()), "pair_embedding", kernels=2)
    return out, resolved


def token_gate(z: torch.Tensor, ids: torch.Tensor, side: torch.Tensor, offset: int) -> torch.Tensor:
    """gelu_tanh(z[t, j]) * side[ids[t], offset + j] for z [tokens, dim], in z's type."""
    z = materialize(z)
    _contig(z, ids, side)
    out = torch.empty_like(z)
    _check(library().vosti_token_gate(_p(z), _is_f32(z), _p(ids), _p(side), _is_f32(side), ctypes.c_int64(side.shape[1]),
                                      offset, z.shape[1], side.shape[0], _p(out), z.shape[0], _stream()), "token_gate")
    return out


# ---------------------------------------------------------------- attention with bias and sink
def qkv_store(qkv: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *, nq: int, nkv: int,
              dk: int, dv: int, page_size: int, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
              temp_coef: float, temp_every: int, status: torch.Tensor,
              freq: Optional[torch.Tensor] = None, magnitude: float = 1.0,
              v_first: Optional[torch.Tensor] = None, v_mix: float = 0.0) -> torch.Tensor:
    """After a q | k | v projection: the queries times their temperature
    (1 + coef * ln(floor((p + 1) / every) + 1), 1 if coef is 0) are returned [tokens, nq * dk];
    keys and values go to their cache slots (caches of different widths). With `freq` (float32
    [n]) the first 2n elements of every query and key head are first turned in pairs (i, i + n) by
    the angle position * freq[i], cos and sin multiplied by `magnitude`. With `v_first` (the values
    [tokens, nkv * dv] another layer made of the same tokens; rows may be strided) the values
    stored are (1 - v_mix) * v + v_mix * v_first, formed in float32 and rounded once."""
    qkv = materialize(qkv)
    _contig(qkv, k_cache, v_cache, positions, slot_mapping, freq)
    flag = _same_dtype(qkv, k_cache, v_cache)
    tokens = qkv.shape[0]
    if freq is not None and freq.dtype != torch.float32:
        raise KernelError("qkv_store: rotation frequencies are float32")
    if qkv.shape[1] != nq * dk + nkv * (dk + dv):
        raise KernelError("qkv_store: input width does not match the head counts")
    if v_first is not None and (v_first.dtype != qkv.dtype or tuple(v_first.shape) != (tokens, nkv * dv)
                                or v_first.stride(1) != 1):
        raise KernelError("qkv_store: the values to mix in are [tokens, nkv * dv] of the projection's type")
    q = torch.empty((tokens, nq * dk), dtype=qkv.dtype, device=qkv.device)
    num_slots = 0 if k_cache is None else k_cache.numel() // (nkv * dk)
    _check(library().vosti_qkv_store(_p(qkv), _p(q), _p(k_cache), _p(v_cache), _p(positions), _p(slot_mapping),
                                     ctypes.c_int64(num_slots), page_size, tokens, nq, nkv, dk, dv,
                                     ctypes.c_float(temp_coef), int(temp_every), flag, _p(status), _p(freq),
                                     0 if freq is None else freq.shape[0], ctypes.c_float(magnitude), _p(v_first),
                                     ctypes.c_int64(0 if v_first is None else v_first.stride(0)), ctypes.c_float(v_mix),
                                     _stream()), "qkv_store")
    return q


SINK_SEGMENT = int(_os.environ.get("VOSTI_SINK_SEGMENT", "256"))          # keys per segment when few query rows share the GPU
SINK_SPLIT_MAX_ROWS = 2048  # (token, head) rows up to which the keys are cut into segments


class HeadFinish:
    """What follows a head's softmax-weighted sum before the output projection, in float32 (the
    kernels' HeadFinish): with two score maps a head o = a1 - `lam` * a2; with `unit_norm`
    o / sqrt(mean(o^2) + eps) * out_scale over the head's values; with `gate` ([tokens, >= nq * dv],
    float32 or bfloat16, rows may be strided: a view of a wider product) o * sigmoid(gate)."""

    def __init__(self, *, lam: float = 0.0, unit_norm: bool = False, eps: float = 0.0, out_scale: float = 1.0,
                 gate: Optional[torch.Tensor] = None):
        self.lam, self.unit_norm, self.eps, self.out_scale, self.gate = float(lam), bool(unit_norm), float(eps), float(out_scale), gate
        if gate is not None and (gate.dim() != 2 or gate.stride(1) != 1):
            raise KernelError("head finish: the gate is [tokens, heads * width] with contiguous rows")

    def args(self):
        g = self.gate
        return (ctypes.c_float(self.lam), int(self.unit_norm), ctypes.c_float(self.eps), ctypes.c_float(self.out_scale), _p(g),
                0 if g is None else _is_f32(g), ctypes.c_longlong(0 if g is None else g.stride(0)))


_NO_FINISH = HeadFinish()


def head_finish(a: torch.Tensor, finish: "HeadFinish", *, nq: int, maps: int, dv: int, in_width: Optional[int] = None,
                pair_group: int = 0) -> torch.Tensor:
    """`finish` applied to attention outputs that another kernel wrote, a [tokens, nq * maps * in_width]
    (of every row of `in_width` elements, default dv, the first dv count); returns [tokens, nq * dv].
    `pair_group` 0: head h's maps are rows h * maps + m of a token; r > 0 (maps that ran as heads of
    their own, grouped by kv head with r heads a kv head): rows h + (h // r) * r + m * r."""
    _contig(a)
    tokens = a.shape[0]
    in_width = dv if in_width is None else in_width
    if a.shape[1] != nq * maps * in_width:
        raise KernelError("head_finish: the input's width does not match heads, maps and width")
    out = torch.empty((tokens, nq * dv), dtype=a.dtype, device=a.device)
    _check(library().vosti_head_finish(_p(a), _p(out), tokens, nq, maps, dv, in_width, pair_group, *finish.args(), _is_f32(a),
                                       _stream()), "head_finish")
    return out


def qkv_heads(proj: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *, nq: int, nkv: int,
              maps: int = 1, dk: int, dv: int, page_size: int, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
              out_dtype: torch.dtype, status: torch.Tensor, bias: Optional[torch.Tensor] = None,
              q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, eps: float = 0.0,
              freq: Optional[torch.Tensor] = None, interleaved: bool = False, magnitude: float = 1.0,
              expanded_width: int = 0) -> torch.Tensor:
    """After a q | k | v projection `proj` [tokens, >= (nq + nkv) * maps * dk + nkv * dv] (float32 or the
    serving type; further columns may follow): `bias` (float32, over the q | k | v columns) is
    added; every query and key head is RMS-normed with the weights `q_norm` / `k_norm` [dk] shared
    by all heads; the first 2 * len(freq) elements of those heads turn by position * freq[i],
    element i with i + len(freq), or 2i with 2i + 1 if `interleaved` (cos and sin times
    `magnitude`); all in float32, rounded once to `out_dtype`. The queries are returned
    [tokens, nq * maps * dk]; keys and values go to their cache slots ([pages, nkv, page_size,
    maps * dk] and [pages, nkv, page_size, dv]). `maps` > 1: the projection holds `maps` query heads
    a head and `maps` key heads a kv head, head by head. `proj` may be a float32 product's unsummed
    K splits (`PartialSum`): the kernel adds them in split order, and the call returns (queries, the
    summed float32 columns that follow q | k | v, or None if there are none). `expanded_width` D > 0 lays every map out as
    a head of its own, D wide, for kernels that know one map a head and one width: queries
    [tokens, nq * maps * D] and caches [pages, nkv * maps, page_size, D] with zeros after a head's own
    elements, a kv head's values stored once for each of its maps."""
    splits, extra = 1, None
    width = (nq + nkv) * maps * dk + nkv * dv
    if isinstance(proj, PartialSum) and proj.dtype == torch.float32:
        # the product's unsummed K splits: added here; columns after q | k | v (a gate) come back summed
        proj.check()
        splits, rows, full = proj.splits, proj.rows, proj.width
        proj = proj.partial[: splits * rows * full].view(splits * rows, full)[:rows]
        if full > width:
            extra = torch.empty((rows, full - width), dtype=torch.float32, device=proj.device)
    proj = materialize(proj)
    _contig(k_cache, v_cache, positions, slot_mapping, freq, bias, q_norm, k_norm)
    tokens = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < width:
        raise KernelError("qkv_heads: the projection is [tokens, >= q | k | v columns] with contiguous rows")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != width):
        raise KernelError("qkv_heads: the bias is float32 over the q | k | v columns")
    if freq is not None and freq.dtype != torch.float32:
        raise KernelError("qkv_heads: rotation frequencies are float32")
    norm_flag = 0
    if q_norm is not None or k_norm is not None:
        norm_flag = _is_f32(q_norm if q_norm is not None else k_norm)
        if q_norm is not None and k_norm is not None and _is_f32(q_norm) != _is_f32(k_norm):
            raise KernelError("qkv_heads: q and k norm weights must share a dtype")
    for cache in (k_cache, v_cache):
        if cache is not None and cache.dtype != out_dtype:
            raise KernelError("qkv_heads: the caches hold the output type")
    D = int(expanded_width)
    if D and (D < dk or D < dv):
        raise KernelError("qkv_heads: expanded heads are at least as wide as the key and value heads")
    q = torch.empty((tokens, nq * maps * (D or dk)), dtype=out_dtype, device=proj.device)
    num_slots = 0 if k_cache is None else k_cache.numel() // (nkv * maps * (D or dk))
    _check(library().vosti_qkv_heads(_p(proj), _is_f32(proj), ctypes.c_longlong(proj.stride(0)), _p(bias), _p(q), _p(k_cache),
                                     _p(v_cache), _p(positions), _p(slot_mapping), ctypes.c_int64(num_slots), page_size, tokens,
                                     nq, nkv, maps, dk, dv, _p(q_norm), _p(k_norm), norm_flag, ctypes.c_float(eps), _p(freq),
                                     0 if freq is None else freq.shape[0], int(bool(interleaved)), ctypes.c_float(magnitude),
                                     int(D > 0), D, D, splits, _p(extra), 0 if extra is None else extra.shape[1],
                                     1 if out_dtype == torch.float32 else 0, _p(status), _stream()), "qkv_heads")
    return q if splits == 1 else (q, extra)


def _attention_sink_rows(ctx, q, k_cache, v_cache, out, group, *, token_list, count, nq, nkv, dk, dv, scale, window,
                         bias, sink, maps=1, finish=None) -> None:
    """The CUDA-core kernel over `count` rows of the step (all of them if `token_list` is None)."""
    flag = _same_dtype(q, k_cache, v_cache)
    num_pages = k_cache.numel() // (group.page_size * nkv * maps * dk)
    segments, scratch = 1, None
    if count * nq <= SINK_SPLIT_MAX_ROWS and ctx.max_kv_len > SINK_SEGMENT:
        segments = -(-ctx.max_kv_len // SINK_SEGMENT)
        scratch = _workspace(q.device, count * nq * segments * maps * (dv + 2))
    _check(library().vosti_attention_maps(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(ctx.positions), _p(ctx.request_of), _p(group.block_table),
        group.block_table.shape[1], group.page_size, num_pages, _p(token_list), count, nq, nkv, maps, dk, dv,
        ctypes.c_float(scale), window, _p(bias), 0 if bias is None else bias.shape[1] - 1, _p(sink), _p(scratch),
        SINK_SEGMENT, segments, *(finish or _NO_FINISH).args(), flag, _p(ctx.status), _stream()), "attention_sink",
        kernels=2 if segments > 1 else 1)


def attention_sink(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, *, nq: int, nkv: int,
                   dk: int, dv: int, scale: float, window: int, bias: Optional[torch.Tensor],
                   sink: Optional[torch.Tensor], chunk: int = 0, maps: int = 1,
                   finish: Optional["HeadFinish"] = None) -> torch.Tensor:
    """Causal attention of every query row over its request's cached keys (the last `window` of
    them, or with `chunk` those of the query's own chunk of positions), with an optional bias
    table float32 [nq, distances] (base-2 units, the last column serving every larger distance)
    and an optional sink logit per head (float32 [nq], natural units). Returns [tokens, nq * dv].
    With `maps` = 2 a head has two score maps (queries [tokens, nq, 2, dk], the key cache's entries
    2 * dk wide) over the same values; `finish` (a `HeadFinish`) says how they are combined and what
    else follows the softmax (unit norm, gate).
    bfloat16 with one map and equal key and value widths of 64 or 128 (pages of a multiple of 16
    tokens, at most 16 query heads per kv head): long rows run on the tensor-memory kernel and
    requests that bring a few tokens on the split-key decode kernels, as Qwen3's do, both with the
    bias and the sink, and `finish` is a kernel of its own after them. Everything else runs on the
    CUDA-core kernel, with the keys cut into segments when the step has few rows, and `finish` is
    its last step."""
    _contig(q, k_cache, v_cache, bias, sink)
    tokens = q.shape[0]
    out = torch.empty((tokens, nq * dv), dtype=q.dtype, device=q.device)
    if chunk < 0 or window < 0 or (chunk and window):
        raise KernelError("attention_sink: a window or a chunk, not both, and neither negative")
    window = -chunk if chunk else window            # the kernels take a chunk as a negative window
    common = dict(nq=nq, nkv=nkv, dk=dk, dv=dv, scale=scale, window=window, bias=bias, sink=sink)
    lib = library()
    tensor_memory = (q.dtype == torch.bfloat16 and dk == dv and nq // nkv <= 16 and maps == 1
                     and lib.vosti_attention_prefill_tc_supported(dk, group.page_size))
    if not tensor_memory or getattr(ctx, "layout", None) is None or "attention" not in ctx.layout:
        _attention_sink_rows(ctx, q, k_cache, v_cache, out, group, token_list=None, count=tokens, maps=maps, finish=finish, **common)
        return out
    # as for `attention`: requests that bring a few tokens one query at a time with split keys,
    # longer portions tile by tile on the tensor-memory kernel (the step's work lists)
    lists = ctx.layout["attention"]
    num_pages = k_cache.numel() // (group.page_size * nkv * dk)
    bias_last = 0 if bias is None else bias.shape[1] - 1
    if lists["num_short_tokens"]:
        count = lists["num_short_tokens"]
        lib.vosti_attention_decode_scratch.restype = ctypes.c_int64
        scratch = _workspace(q.device, lib.vosti_attention_decode_scratch(count, nq, nkv, dk, ctx.max_kv_len))
        arrivals = _counters(q.device, count * nkv)
        _check(lib.vosti_attention_decode_biased(
            _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scratch), ctypes.c_int64(scratch.numel()), _p(arrivals),
            _p(ctx.extras.get("attention.short_tokens")), count, tokens, _p(ctx.positions), _p(ctx.request_of),
            _p(group.block_table), group.block_table.shape[1], group.page_size, num_pages, nq, nkv, dk, ctx.max_kv_len,
            ctypes.c_float(scale), window, _p(bias), bias_last, _p(sink), _p(ctx.status), _stream()),
            "attention_decode_biased")
    if lists["num_long_rows"]:
        _check(lib.vosti_attention_prefill_tc_biased(
            _p(q), _p(k_cache), _p(v_cache), _p(out), _p(ctx.extras.get("attention.long_rows")), lists["num_long_rows"],
            _p(ctx.cu_q), _p(ctx.kv_len), _p(group.block_table), group.block_table.shape[1], group.page_size, num_pages,
            nq, nkv, dk, lists["max_long_q_len"], tokens, ctypes.c_float(scale), window, _p(bias), bias_last, _p(sink),
            _p(ctx.status), _stream()), "attention_prefill_tc_biased")
    if finish is not None:
        return head_finish(out, finish, nq=nq, maps=1, dv=dv)
    return out


def attention_heads_supported(dtype: torch.dtype, width: int, group: int) -> bool:
    """Whether heads of equal key and value width `width` with `group` query heads a kv head can run on
    the tensor-core attention kernels (given pages of a multiple of 16 tokens)."""
    return bool(dtype == torch.bfloat16 and group <= 16 and library().vosti_attention_prefill_tc_supported(width, 16))


# ---------------------------------------------------------------- layer norm over the stream
class DeferredNormed:
    """A sublayer's output [rows, width] that is still to be layer-normed (weight, optional bias),
    multiplied element by element by an optional `scale` vector and added to the float32 residual
    stream: the kernel that next reads the stream (`layer_norm_stream`) does all of it."""

    def __init__(self, y, weight: torch.Tensor, bias: Optional[torch.Tensor], scale: Optional[torch.Tensor], eps: float):
        self.y = materialize(y)
        self.weight, self.bias, self.scale, self.eps = weight, bias, scale, float(eps)
        small = [t for t in (weight, bias, scale) if t is not None]
        if len({t.dtype for t in small}) > 1:
            self.weight, self.bias, self.scale = (None if t is None else t.float() for t in (weight, bias, scale))
        self.shape = tuple(self.y.shape)

    def rows(self, index: torch.Tensor, status: torch.Tensor) -> "DeferredNormed":
        """The same for the rows `index` names."""
        return DeferredNormed(gather_rows(self.y, index, status), self.weight, self.bias, self.scale, self.eps)


def layer_norm_stream(x, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
                      out_dtype: Optional[torch.dtype], *, stream: Optional[torch.Tensor] = None,
                      stream_out: Optional[torch.Tensor] = None):
    """Layer norm of s = stream + x over a float32 residual stream: (s - mean) / sqrt(var + eps) *
    weight + bias in float32 (var: the mean of the squared deviations), rounded to `out_dtype`; s
    goes to `stream_out` (float32, may be `stream`). x is a tensor, None, or a `DeferredNormed`,
    which is normed and scaled on the way in. Without `out_dtype` only the sum is stored."""
    y = wy = by = sy = None
    eps_y = 0.0
    if isinstance(x, DeferredNormed):
        y, wy, by, sy, eps_y = x.y, x.weight, x.bias, x.scale, x.eps
    elif x is not None:
        y = materialize(x)
    like = stream if stream is not None else y
    _contig(stream, stream_out, y, wy, by, sy, weight, bias)
    if stream is not None and stream.dtype != torch.float32 or stream_out is not None and stream_out.dtype != torch.float32:
        raise KernelError("layer_norm_stream: the residual stream is float32")
    if bias is not None and bias.dtype != weight.dtype:
        raise KernelError("layer_norm_stream: weight and bias must share a dtype")
    rows, width = like.shape
    out = None if out_dtype is None else torch.empty((rows, width), dtype=out_dtype, device=like.device)
    _check(library().vosti_layer_norm_stream(
        _p(stream), _p(y), 0 if y is None else _is_f32(y), _p(wy), _p(by), _p(sy), 0 if wy is None else _is_f32(wy),
        ctypes.c_float(eps_y), _p(stream_out), _p(weight), _p(bias), 0 if weight is None else _is_f32(weight),
        ctypes.c_float(eps), _p(out), 0 if out is None else _is_f32(out), rows, width, _stream()), "layer_norm_stream")
    return out


# ---------------------------------------------------------------- latent attention
def latent_prep(proj: torch.Tensor, qk: torch.Tensor, c_cache: Optional[torch.Tensor], r_cache: Optional[torch.Tensor],
                norm_w: torch.Tensor, eps: float, ctx, slot_mapping: Optional[torch.Tensor], *, heads: int, dim: int, rot: int,
                rank: int, freq: Optional[torch.Tensor], magnitude: float) -> torch.Tensor:
    """After the q | down | gate projection (csrc/attention_latent.cu): the rotated part of every
    query head goes to the last `rot` columns of qk [tokens, heads, rank + rot]; the latent
    (root-mean-square normed with `norm_w`) and the rotated shared key part go to their cache
    slots; returns sigmoid(gate) float32 [tokens, heads]."""
    proj = materialize(proj)
    _contig(proj, qk, c_cache, r_cache, norm_w, slot_mapping, freq)
    flag = _same_dtype(proj, qk, c_cache, r_cache)
    tokens = proj.shape[0]
    if proj.shape[1] != heads * (dim + rot) + rank + rot + heads or tuple(qk.shape) != (tokens, heads, rank + rot):
        raise KernelError("latent_prep: widths do not match the head sizes")
    gate = torch.empty((tokens, heads), dtype=torch.float32, device=proj.device)
    num_slots = 0 if c_cache is None else c_cache.numel() // rank
    _check(library().vosti_latent_prep(_p(proj), _p(qk), _p(gate), _p(c_cache), _p(r_cache), _p(norm_w), _is_f32(norm_w),
                                       ctypes.c_float(eps), _p(ctx.positions), _p(slot_mapping), ctypes.c_int64(num_slots),
                                       tokens, heads, dim, rot, rank, _p(freq), ctypes.c_float(magnitude), flag,
                                       _p(ctx.status), _stream()), "latent_prep")
    return gate


def head_project(x: torch.Tensor, m: torch.Tensor, y: torch.Tensor, *, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, h, :] = gate[t, h] * (x[t, h, :] @ m[h]) with float32 sums. x [tokens, heads, in],
    m [heads, in, out] and y [tokens, heads, out] may be strided views (unit stride along x's and
    y's last axis); gate float32 [tokens, heads]. A bfloat16 m with a contiguous inner or output
    axis and strides in multiples of 8 runs on the tensor cores (a float32 x as two bfloat16
    terms); everything else on the CUDA cores in float32."""
    tokens, heads, inner = x.shape
    if tuple(m.shape[:2]) != (heads, inner) or tuple(y.shape) != (tokens, heads, m.shape[2]):
        raise KernelError("head_project: shapes do not fit")
    if tokens and (x.stride(2) != 1 or y.stride(2) != 1):
        raise KernelError("head_project: the last axis of x and y must be contiguous")
    _contig(gate)
    lib = library()
    if (tokens and m.dtype == torch.bfloat16 and x.dtype in (torch.bfloat16, torch.float32)
            and y.dtype in (torch.bfloat16, torch.float32) and x.data_ptr() % 16 == 0 and m.data_ptr() % 16 == 0
            and y.data_ptr() % 8 == 0
            and lib.vosti_head_project_mma_fits(ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)), _is_f32(x),
                                                ctypes.c_int64(m.stride(0)), ctypes.c_int64(m.stride(1)),
                                                ctypes.c_int64(m.stride(2)), ctypes.c_int64(y.stride(0)),
                                                ctypes.c_int64(y.stride(1)), inner, m.shape[2])):
        _check(lib.vosti_head_project_mma(
            _p(x), _is_f32(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)), _p(m), ctypes.c_int64(m.stride(0)),
            ctypes.c_int64(m.stride(1)), ctypes.c_int64(m.stride(2)), _p(gate), _p(y), _is_f32(y), ctypes.c_int64(y.stride(0)),
            ctypes.c_int64(y.stride(1)), tokens, heads, inner, m.shape[2], _stream()), "head_project_mma")
        return y
    _check(lib.vosti_head_project(
        _p(x), _is_f32(x), ctypes.c_int64(x.stride(0)), ctypes.c_int64(x.stride(1)), _p(m), _is_f32(m),
        ctypes.c_int64(m.stride(0)), ctypes.c_int64(m.stride(1)), ctypes.c_int64(m.stride(2)), _p(gate), _p(y), _is_f32(y),
        ctypes.c_int64(y.stride(0)), ctypes.c_int64(y.stride(1)), tokens, heads, inner, m.shape[2], _stream()), "head_project")
    return y


LATENT_SEGMENT = 256           # keys per segment when few query rows share the GPU
LATENT_SPLIT_MAX_ROWS = 2048   # (token, head) rows up to which the keys are cut into segments
LATENT_MMA_SEGMENT = 128       # the same for the tensor-core kernel, whose CTA takes 16 or 32 rows
LATENT_MMA_SPLIT_BELOW = 296   # CTAs (two per SM) below which it cuts the keys


def latent_attend(ctx, qk: torch.Tensor, c_cache: torch.Tensor, r_cache: torch.Tensor, group, *, scale: float,
                  window: int = 0) -> torch.Tensor:
    """Causal softmax attention of every (token, head) row of qk [tokens, heads, rank + rot] over the
    cached latents [pages, 1, page_size, rank] and shared rotated key parts [.., rot] of its
    request; returns the weighted latents, float32 [tokens, heads, rank]. bfloat16 with a rank of
    128, 256 or 512 and a rotated part in multiples of 32 runs on the tensor cores
    (csrc/attention_latent_mma.cu), everything else on the CUDA cores (csrc/attention_latent.cu)."""
    _contig(qk, c_cache, r_cache)
    flag = _same_dtype(qk, c_cache, r_cache)
    tokens, heads = qk.shape[0], qk.shape[1]
    rank, rot = c_cache.shape[-1], r_cache.shape[-1]
    out = torch.empty((tokens, heads, rank), dtype=torch.float32, device=qk.device)
    num_pages = c_cache.shape[0]
    lib = library()
    segments, scratch = 1, None
    if not flag and window >= 0 and lib.vosti_latent_attend_mma_fits(rank, rot):
        rows = ctx.max_q_len * heads
        ctas = -(-rows // (32 if rows > 16 else 16)) * ctx.num_requests
        if ctas < LATENT_MMA_SPLIT_BELOW and ctx.max_kv_len > LATENT_MMA_SEGMENT:
            segments = -(-ctx.max_kv_len // LATENT_MMA_SEGMENT)
            scratch = _workspace(qk.device, tokens * heads * segments * (rank + 2))
        _check(lib.vosti_latent_attend_mma(
            _p(qk), _p(c_cache), _p(r_cache), _p(out), _p(ctx.positions), _p(ctx.cu_q), _p(group.block_table),
            group.block_table.shape[1], group.page_size, num_pages, ctx.num_requests, ctx.max_q_len, heads, rank, rot,
            ctypes.c_float(scale), window, _p(scratch), LATENT_MMA_SEGMENT, segments, _p(ctx.status), _stream()),
            "latent_attend_mma")
        if segments > 1:
            _check(lib.vosti_latent_merge(_p(scratch), segments, _p(out), tokens, heads, rank, _stream()), "latent_merge")
        return out
    if tokens * heads <= LATENT_SPLIT_MAX_ROWS and ctx.max_kv_len > LATENT_SEGMENT:
        segments = -(-ctx.max_kv_len // LATENT_SEGMENT)
        scratch = _workspace(qk.device, tokens * heads * segments * (rank + 2))
    _check(lib.vosti_latent_attend(
        _p(qk), _p(c_cache), _p(r_cache), _p(out), _p(ctx.positions), _p(ctx.request_of), _p(group.block_table),
        group.block_table.shape[1], group.page_size, num_pages, None, tokens, heads, rank, rot, ctypes.c_float(scale),
        window, _p(scratch), LATENT_SEGMENT, segments, flag, _p(ctx.status), _stream()), "latent_attend",
        kernels=2 if segments > 1 else 1)
    return out


# ---------------------------------------------------------------- selective scan
def scan_conv(xz: torch.Tensor, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], state: torch.Tensor, tail_offset: int,
              ctx, *, inner: int, taps: int) -> torch.Tensor:
    """silu(causal convolution) of the first `inner` columns of xz [tokens, >= inner] per channel
    (csrc/selective_scan.cu); the inputs before a portion come from the tail [taps - 1, inner] kept
    `tail_offset` floats into the request's state slot, which is then moved on."""
    xz = materialize(xz)
    _contig(xz, conv_w, conv_b, state)
    if conv_b is not None and conv_b.dtype != conv_w.dtype or state.dtype != torch.float32:
        raise KernelError("scan_conv: the convolution's tensors share a type and the state is float32")
    tokens = xz.shape[0]
    out = torch.empty((tokens, inner), dtype=xz.dtype, device=xz.device)
    _check(library().vosti_scan_conv(
        _p(xz), ctypes.c_int64(xz.shape[1]), _p(conv_w), _p(conv_b), _is_f32(conv_w), _p(state), ctypes.c_int64(state.shape[1]),
        ctypes.c_int64(tail_offset), _p(ctx.request_of), _p(ctx.cu_q), _p(ctx.state_slots), state.shape[0], ctx.num_requests,
        tokens, inner, taps, _p(out), _is_f32(xz), _p(ctx.status), _stream()), "scan_conv", kernels=2 if taps > 1 else 1)
    return out


def scan_run(x: torch.Tensor, dtp: torch.Tensor, dt_bias: Optional[torch.Tensor], bc: torch.Tensor, a_log: torch.Tensor,
             d_skip: Optional[torch.Tensor], xz: torch.Tensor, state: torch.Tensor, ctx, *, inner: int, states: int) -> torch.Tensor:
    """The selective-scan recurrence over every request's tokens of this step, from and to its state
    slot: x [tokens, inner] (convolved), dtp float32 [tokens, inner] (step sizes before bias and
    softplus), bc float32 [tokens, 2 * states], z = the columns [inner, 2 * inner) of xz. Returns
    (S C + D x) * silu(z) in x's type."""
    _contig(x, dtp, dt_bias, bc, a_log, d_skip, xz, state)
    small = [t for t in (dt_bias, a_log, d_skip) if t is not None]
    if len({t.dtype for t in small}) > 1 or dtp.dtype != torch.float32 or bc.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("scan_run: the small tensors share a type; step sizes, B | C and the state are float32")
    if xz.dtype != x.dtype or xz.shape[1] < 2 * inner or tuple(bc.shape) != (x.shape[0], 2 * states):
        raise KernelError("scan_run: shapes do not fit")
    y = torch.empty_like(x)
    z = xz[:, inner:]
    chunk = library().vosti_scan_chunk(states)
    ws = ws_dt = None
    several = ctx.max_q_len > chunk
    if several:                  # chunks of a long portion run side by side: start states and step-size sums per chunk
        places = x.shape[0] // chunk + ctx.num_requests
        ws = torch.empty((places, inner, states), dtype=torch.float32, device=x.device)
        ws_dt = torch.empty((places, inner), dtype=torch.float32, device=x.device)
    _check(library().vosti_scan_run(
        _p(x), _p(dtp), _p(dt_bias), _p(bc), _p(a_log), _p(d_skip), _is_f32(a_log), _p(z), ctypes.c_int64(xz.shape[1]),
        _p(state), ctypes.c_int64(state.shape[1]), _p(ctx.cu_q), _p(ctx.state_slots), state.shape[0], ctx.num_requests,
        ctx.max_q_len, inner, states, _p(ws), _p(ws_dt), _p(y), _is_f32(x), _p(ctx.status), _stream()), "scan_run",
        kernels=3 if several else 1)
    return y


# ---------------------------------------------------------------- gated delta rule
def delta_prep(proj: torch.Tensor, rates: torch.Tensor, offsets: dict, *, kv_heads: int, heads: int, dk: int, dv: int,
               taps: int, conv_w, a_log, dt_bias, state: torch.Tensor, conv_offset: int, ctx,
               decay_per_head: bool = False, gate_silu: bool = False):
    """Everything between the projections and the recurrence (see csrc/delta_rule.cu): `proj` holds
    the columns q | k | v | beta at `offsets`, `rates` [tokens, heads*dk + heads*dv] the low-rank
    pairs' products (decay rates, then output gates, before their activations). Also moves the
    convolution tail in the requests' state slots on. Returns float32 q, k, v, beta, decay, gate."""
    proj, rates = materialize(proj), materialize(rates)
    small = (conv_w, a_log, dt_bias)
    _contig(proj, rates, state, *small)
    flag = _is_f32(conv_w)
    if any(_is_f32(t) != flag for t in small) or state.dtype != torch.float32:
        raise KernelError("delta_prep: the small tensors must share a dtype and the state is float32")
    tokens, dev = proj.shape[0], proj.device
    if tuple(rates.shape) != (tokens, (heads if decay_per_head else heads * dk) + heads * dv):
        raise KernelError("delta_prep: the rates do not match the head sizes")
    new = lambda width: torch.empty((tokens, width), dtype=torch.float32, device=dev)
    q, k, v = new(kv_heads * dk), new(kv_heads * dk), new(heads * dv)
    beta, decay, gate = new(heads), new(heads * dk), new(heads * dv)
    _check(library().vosti_delta_prep(
        _p(proj), _is_f32(proj), proj.shape[1], offsets["q"], offsets["k"], offsets["v"], offsets["b"], _p(rates),
        _is_f32(rates), kv_heads, heads, dk, dv, taps, _p(conv_w), _p(a_log), _p(dt_bias), flag, _p(state),
        ctypes.c_int64(state.shape[1]), ctypes.c_int64(conv_offset), _p(ctx.request_of), _p(ctx.cu_q),
        _p(ctx.state_slots), state.shape[0], ctx.num_requests, tokens, _p(q), _p(k), _p(v), _p(beta), _p(decay), _p(gate),
        _p(ctx.status), int(decay_per_head), int(gate_silu), _stream()), "delta_prep", kernels=2 if taps > 1 else 1)
    return q, k, v, beta, decay, gate


def delta_scan(q, k, v, beta, decay, state: torch.Tensor, ctx, *, kv_heads: int, heads: int, dk: int, dv: int) -> torch.Tensor:
    """The recurrence over every request's tokens of this step, from and to its state slot;
    returns the read-outs, float32 [tokens, heads * dv]."""
    _contig(q, k, v, beta, decay, state)
    out = torch.empty((q.shape[0], heads * dv), dtype=torch.float32, device=q.device)
    _check(library().vosti_delta_scan(_p(q), _p(k), _p(v), _p(beta), _p(decay), _p(out), _p(state),
                                      ctypes.c_int64(state.shape[1]), _p(ctx.cu_q), _p(ctx.state_slots), state.shape[0],
                                      ctx.num_requests, kv_heads, heads, dk, dv, _stream()), "delta_scan")
    return out


def delta_out(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, *, heads: int, dv: int,
              out_dtype: torch.dtype) -> torch.Tensor:
    """o / sqrt(mean(o^2) + eps) * weight * gate per (token, head), rounded to `out_dtype`; the
    weight is [dv], shared by the heads, or [heads * dv]."""
    _contig(o, gate, weight)
    if weight.numel() not in (dv, heads * dv):
        raise KernelError("delta_out: the weight has one row, or one per head")
    y = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    _check(library().vosti_delta_out(_p(o), _p(gate), _p(weight), _is_f32(weight), _p(y), _is_f32(y), o.shape[0], heads, dv,
                                     ctypes.c_float(eps), int(weight.numel() != dv), _stream()), "delta_out")
    return y


def tanh_columns(x: torch.Tensor, offset: int, width: int) -> torch.Tensor:
    """tanh(x[:, offset:offset + width]) as a contiguous tensor of x's type."""
    x = materialize(x)
    _contig(x)
    out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    _check(library().vosti_tanh_columns(_p(x), _is_f32(x), x.shape[1], offset, width, _p(out), x.shape[0], _stream()),
           "tanh_columns")
    return out


def general_delta_prep(proj: torch.Tensor, inner: torch.Tensor, offsets: dict, *, heads: int, d: int, w0: torch.Tensor,
                       a_bias: torch.Tensor):
    """Between the projections and the generalized delta rule's recurrence (csrc/delta_rule.cu):
    `proj` holds the columns r | k | v | g | a at `offsets`, `inner` float32 [tokens, heads * d] the
    decay's low-rank product. Returns float32 r, k, v, decay, unit key, removal (rate * unit key), gate."""
    proj, inner = materialize(proj), materialize(inner)
    _contig(proj, inner, w0, a_bias)
    if inner.dtype != torch.float32 or _is_f32(w0) != _is_f32(a_bias) or tuple(inner.shape) != (proj.shape[0], heads * d):
        raise KernelError("general_delta_prep: the low-rank product is float32 [tokens, heads * d]; the biases share a type")
    tokens = proj.shape[0]
    outs = [torch.empty((tokens, heads * d), dtype=torch.float32, device=proj.device) for _ in range(7)]
    _check(library().vosti_general_delta_prep(
        _p(proj), _is_f32(proj), proj.shape[1], offsets["r"], offsets["k"], offsets["v"], offsets["g"], offsets["a"],
        _p(inner), _p(w0), _p(a_bias), _is_f32(w0), heads, d, tokens, *[_p(t) for t in outs], _stream()), "general_delta_prep")
    return outs


def general_delta_scan(r, k, v, decay, unit, removal, state: torch.Tensor, ctx, *, heads: int, d: int) -> torch.Tensor:
    """The generalized rule's recurrence over every request's tokens of this step, from and to its
    state slot; returns the read-outs, float32 [tokens, heads * d]."""
    _contig(r, k, v, decay, unit, removal, state)
    out = torch.empty((r.shape[0], heads * d), dtype=torch.float32, device=r.device)
    _check(library().vosti_general_delta_scan(_p(r), _p(k), _p(v), _p(decay), _p(unit), _p(removal), _p(out), _p(state),
                                              ctypes.c_int64(state.shape[1]), _p(ctx.cu_q), _p(ctx.state_slots),
                                              state.shape[0], ctx.num_requests, heads, d, d, _stream()), "general_delta_scan")
    return out


# ---------------------------------------------------------------- mixture of experts
def moe_route(logits: torch.Tensor, top: int, *, over_all: bool = False, scale: float = 1.0):
    """The `top` largest of each row of float32 router logits: (expert ids int32 [tokens, top],
    their weights float32 [tokens, top], the same weights as a dense [tokens, experts]). The
    weights are the softmax over the chosen logits, or with `over_all` the chosen experts' shares
    of a softmax over all experts divided by their sum (+ 1e-20); both times `scale`."""
    if logits.dtype != torch.float32:
        raise KernelError("moe_route: router logits are float32")
    _contig(logits)
    tokens, experts = logits.shape
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    dense = torch.empty((tokens, experts), dtype=torch.float32, device=logits.device)
    _check(library().vosti_moe_route(_p(logits), tokens, experts, top, _p(chosen), _p(weights), _p(dense), int(over_all),
                                     ctypes.c_float(scale), _stream()), "moe_route")
    return chosen, weights, dense


def moe_router(x: torch.Tensor, router: torch.Tensor, top: int, *, over_all: bool = False, scale: float = 1.0,
               want_logits: bool = False):
    """The router's product x @ router.T (float32 arithmetic, router float32 [experts, k]) and
    `moe_route` of it in one kernel: (chosen, weights, dense), and the logits too if asked for."""
    x = materialize(x)
    _contig(x, router)
    if router.dtype != torch.float32 or router.shape[1] != x.shape[1]:
        raise KernelError("moe_router: the router is float32 [experts, k]")
    tokens, experts = x.shape[0], router.shape[0]
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    dense = torch.empty((tokens, experts), dtype=torch.float32, device=x.device)
    logits = torch.empty((tokens, experts), dtype=torch.float32, device=x.device) if want_logits else None
    _check(library().vosti_moe_router(_p(x), _is_f32(x), _p(router), tokens, experts, x.shape[1], top, _p(chosen), _p(weights),
                                      _p(dense), _p(logits), int(over_all), ctypes.c_float(scale), _stream()), "moe_router")
    return (chosen, weights, dense, logits) if want_logits else (chosen, weights, dense)


def moe_router_scored(x: torch.Tensor, router: torch.Tensor, top: int, *, identity: int = 0,
                      correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, gate_row: bool = False,
                      scale: float = 1.0, want_logits: bool = False):
    """Router product and choice by corrected scores in one kernel. `router` is float32
    [routed + (1 if gate_row), k]: `routed` rows take part in the choice, of which the last
    `identity` are experts that return their input. s = softmax over the routed logits; rows are
    chosen by s + correction (float32 [routed]) inside the `keep` best of `groups` equal groups of
    neighbouring rows (a group's score: its largest corrected score); weights = the chosen rows' s
    divided by their sum (+ 1e-20), times `scale`. Returns (chosen int32 [tokens, top], weights
    float32 [tokens, top], dense float32 [tokens, routed - identity + (1 if gate_row)], ident float32
    [tokens] or None): dense holds the chosen experts' weights and, with `gate_row`, in its last
    column the sigmoid of the gate row's logit; ident is the sum of the chosen identity experts' weights."""
    x = materialize(x)
    _contig(x, router, correction)
    rows = router.shape[0]
    routed = rows - int(gate_row)
    if router.dtype != torch.float32 or router.shape[1] != x.shape[1]:
        raise KernelError("moe_router: the router is float32 [rows, k]")
    if correction is not None and (correction.dtype != torch.float32 or correction.shape[0] != routed):
        raise KernelError("moe_router: the correction is float32 [routed]")
    tokens = x.shape[0]
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    dense = torch.empty((tokens, routed - identity + int(gate_row)), dtype=torch.float32, device=x.device)
    ident = torch.empty((tokens,), dtype=torch.float32, device=x.device) if identity else None
    logits = torch.empty((tokens, rows), dtype=torch.float32, device=x.device) if want_logits else None
    _check(library().vosti_moe_router_scored(_p(x), _is_f32(x), _p(router), tokens, routed, identity, x.shape[1], top,
                                             _p(correction), groups, keep, int(gate_row), ctypes.c_float(scale), _p(chosen),
                                             _p(weights), _p(dense), _p(ident), _p(logits), _stream()), "moe_router_scored")
    return (chosen, weights, dense, ident, logits) if want_logits else (chosen, weights, dense, ident)


MOE_ACTIVATIONS = {None: 0, "gelu": 1, "relu2": 2}


def moe_scale(act: torch.Tensor, dense: Optional[torch.Tensor], ff: int, *, gelu: bool = False,
              activation: Optional[str] = None, tail: int = 0) -> torch.Tensor:
    """act[t, e * ff + i] <- f(act[t, e * ff + i]) * dense[t, e], in place; f is the exact GELU with
    `gelu` (or `activation` "gelu"), the square of relu with `activation` "relu2", else the identity;
    without `dense` the activation alone. With `tail` the row ends in one more slice of `tail`
    columns, weighted by dense's last column."""
    _contig(act, dense)
    mode = 1 if gelu else MOE_ACTIVATIONS[activation]
    if tail == 0 and mode < 2:
        experts = dense.shape[1] if dense is not None else act.shape[1] // ff
        _check(library().vosti_moe_scale(_p(act), _p(dense), act.shape[0], experts, ff, _is_f32(act), mode, _stream()),
               "moe_scale")
        return act
    experts = (act.shape[1] - tail) // ff
    if experts * ff + tail != act.shape[1] or (dense is not None and dense.shape[1] != experts + (1 if tail else 0)):
        raise KernelError("moe_scale: the activation's width does not match the experts, their width and the tail")
    _check(library().vosti_moe_scale_tail(_p(act), _p(dense), act.shape[0], experts, ff, tail, _is_f32(act), mode, _stream()),
           "moe_scale")
    return act


def moe_identity(y: torch.Tensor, coeff: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """y[t] += coeff[t] * x[t] in place (y float32): the share of experts that return their input."""
    _contig(y, coeff, x)
    if y.dtype != torch.float32 or coeff.dtype != torch.float32 or tuple(x.shape) != tuple(y.shape):
        raise KernelError("moe_identity: y and the coefficients are float32, x has y's shape")
    _check(library().vosti_moe_identity(_p(y), _p(coeff), _p(x), _is_f32(x), y.shape[0], y.shape[1], _stream()), "moe_identity")
    return y


def moe_group(chosen: torch.Tensor, experts: int):
    """Sort the (token, pick) pairs of `chosen` int32 [tokens, top] by expert, keeping their order
    inside an expert: (offsets int32 [experts + 1] of every expert's run, rows int32 [pairs] the
    token at each sorted place, where int32 [tokens, top] the sorted place of every pair)."""
    _contig(chosen)
    tokens, top = chosen.shape
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=chosen.device)
    rows = torch.empty((tokens * top,), dtype=torch.int32, device=chosen.device)
    where = torch.empty((tokens, top), dtype=torch.int32, device=chosen.device)
    _check(library().vosti_moe_group(_p(chosen), tokens, top, experts, _p(offsets), _p(rows), _p(where), _stream()),
           "moe_group")
    return offsets, rows, where


def moe_combine(y: torch.Tensor, where: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[where[t, k]], float32."""
    _contig(y, where, weights)
    if y.dtype != torch.float32 or weights.dtype != torch.float32:
        raise KernelError("moe_combine: the experts' outputs and the weights are float32")
    tokens, top = where.shape
    out = torch.empty((tokens, y.shape[1]), dtype=torch.float32, device=y.device)
    _check(library().vosti_moe_combine(_p(y), _p(where), _p(weights), _p(out), tokens, top, y.shape[1], _stream()),
           "moe_combine")
    return out
