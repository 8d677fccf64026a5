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
              feedback: Optional[tuple] = None, scale: float = 1.0) -> torch.Tensor:
    """table[ids] * scale. `feedback` = (source, values), int32: row t takes values[source[t]] as
    its id where source[t] >= 0 (a token sampled on the device that the host has not read yet)."""
    _contig(ids, table)
    source, values = feedback if feedback is not None else (None, None)
    if source is not None:
        _contig(source, values)
        assert source.shape[0] == ids.shape[0] and source.dtype == values.dtype == torch.int32
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
    return x.materialize() if isinstance(x, PartialSum) else x


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
            swiglu: bool = False, allow_partial: bool = False):
    """y = x @ w.T on the tensor cores (bfloat16 operands, float32 accumulation); w is a
    [features, k] tensor or a `PackedWeight`. With `swiglu` the rows of w are blocks of 16 gate
    rows followed by their 16 up rows and y = silu(gate) * up has half as many columns."""
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
        epilogue, width = EPI_SWIGLU, features // 2
        if out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the fused SiLU*up epilogue writes bfloat16")
    else:
        epilogue, width = (EPI_F32 if out_dtype == torch.float32 else EPI_BF16), features
    global _SPLIT_GENERATION
    lib = library()
    splits = lib.vosti_gemm_tc_splits(tokens, features, k)
    elems = splits * tokens * features if splits > 1 else 0
    ws = _workspace(x.device, elems, "split_k") if elems else None
    defer = bool(allow_partial and splits > 1 and epilogue == EPI_BF16)
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
