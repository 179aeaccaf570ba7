"""Python faces of the CUDA kernels in `csrc/`.

Every function here checks device, dtype, shape and contiguity of what it is given,
then passes raw pointers and the current CUDA stream to an `extern "C"` launcher loaded
by `csrc.build`.  There is no CPU path and no library fallback: a tensor on the CPU, a
missing compiler or a failed launch raises.  Matrix products of 16-bit operands with more
than 64 rows (prompt portions), except the one with the gate in its epilogue, go to cuBLAS
through `torch.mm` (a library product, as in the reference, whose every product is XLA's);
every other operation on the forward path, the products of decode steps among them, is a
kernel of this package.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build as _build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
STATUS_BITS = {1: "token id outside the embedding table", 2: "page id outside the pool or missing from the block table",
               4: "row index outside the batch", 8: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


class PartialSum:
    """A result [n, width] that is given as `parts` [S, n, width] float32 and is their sum over S: what a
    product leaves whose k was cut into S parts for an even load (`linear(..., parts_ok=True)`).  `rmsnorm`
    and `residual_add` take it as `delta` and `swiglu` as its input and add the parts, in order, as they
    read them; `tensor()` adds them up for any other reader."""

    def __init__(self, parts: torch.Tensor):
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def device(self):
        return self.parts.device

    def tensor(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.zeros(tuple(self.shape), dtype=torch.float32, device=self.device)
        residual_add(out, self)
        return out if dtype == torch.float32 else out.to(dtype)


class PickedRows:
    """A result [n, width] given as rows of `rows` [m, width] to be picked and weighted: row r of the result is
    sum_s coef[r, s] * rows[pick[r, s]] (32-bit, s ascending): what a routed feed-forward leaves (its experts'
    outputs in the order of the experts, and for every token where its chosen experts' rows are and what they
    weigh).  `branch_norm_add` adds the rows up as it reads them; `tensor()` does it for any other reader."""

    def __init__(self, rows: torch.Tensor, pick: torch.Tensor, coef: torch.Tensor):
        self.rows, self.pick, self.coef = rows, pick, coef

    @property
    def shape(self):
        return (self.pick.shape[0], self.rows.shape[1])

    @property
    def device(self):
        return self.rows.device

    def tensor(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _cuda(self.rows, "rows"); _cuda(self.pick, "pick", torch.int32); _cuda(self.coef, "coef", torch.float32)
        n, width = self.shape
        out = torch.empty((n, width), dtype=torch.float32, device=self.device)
        f = _fn("branch_norm", "jv_pick_rows_sum", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
                                                    c_int, c_void_p, c_void_p])
        _check(f(self.rows.data_ptr(), _code(self.rows, "rows"), self.pick.data_ptr(), self.coef.data_ptr(),
                 self.pick.shape[1], self.rows.shape[0], out.data_ptr(), n, width, _status_ptr(self.device), _stream()),
               "pick_rows_sum")
        return out if dtype == torch.float32 else out.to(dtype)


_fn_cache: dict[tuple[str, str], object] = {}
launch_count = 0     # kernels of this package launched so far (library products are not counted)
_status: dict[int, torch.Tensor] = {}


def _fn(lib: str, name: str, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(_build.load(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle: asked for before every launch, so by the short way where torch has one."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str, launches: int = 1) -> None:
    if rc == 0:
        global launch_count
        launch_count += launches
        return
    if rc == 2:
        raise KernelError(f"{what}: these sizes are outside what the kernel handles")
    raise KernelError(f"{what}: the launch failed ({torch.cuda.get_device_name()}; "
                      f"the kernels are built for sm_100a only)")


def _cuda(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _code(t: torch.Tensor, name: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def status_word(device=None) -> torch.Tensor:
    """The int32 word (one per device) in which kernels record indices outside their tables."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = w
    return w


_status_ptrs: dict[int, int] = {}


def _status_ptr(device: torch.device) -> int:
    """Address of the status word of a tensor's device (what every launcher is given), without building anything."""
    ptr = _status_ptrs.get(device.index)
    if ptr is None:
        ptr = _status_ptrs[device.index] = status_word(device).data_ptr()
    return ptr


def raise_on_status(value: int) -> None:
    if value:
        msgs = [m for bit, m in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel met " + "; ".join(msgs) + f" (status {value})")


def clear_status(device=None) -> None:
    """Zeroes the status word and what a kernel that gave up may have left half done: the arrival counters of
    the split decode attention (a block that leaves on a bounded wait never counts itself, so its row's
    counter would stay short of the total for every later launch)."""
    w = status_word(device)
    w.zero_()
    buf = _counters.get(w.device.index)
    if buf is not None:
        buf.zero_()


def check_status(device=None) -> None:
    """Reads the status word (a device synchronisation) and raises if a kernel set it."""
    w = status_word(device)
    v = int(w.item())
    if v:
        clear_status(device)
        raise_on_status(v)


# NVTX ranges around the parts of a step (JAX_VLLM_B200_NVTX=1): a profiler's timeline then shows which kernels belong
# to which layer and part.  Off by default: `trace_range` then returns one shared object that does nothing.
TRACE_RANGES = os.environ.get("JAX_VLLM_B200_NVTX", "0") not in ("", "0")


class _NoRange:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _NvtxRange:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


_NO_RANGE = _NoRange()


def trace_range(name: str):
    """A context manager that brackets what runs inside it with an NVTX range of that name, if ranges are on."""
    return _NvtxRange(name) if TRACE_RANGES else _NO_RANGE


def wait_probe(cycles: int, arrive: bool, device=None) -> tuple:
    """Runs the bounded wait of the TMA and tcgen05 kernels alone (csrc/wait_probe.cu): one barrier that a thread
    arrives on (`arrive`) or that nothing ever arrives on, waited for at most `cycles` clocks.  Returns
    (succeeded, clocks spent).  A wait that ran out leaves its bit in the status word, as in the product kernels:
    `check_status` raises afterwards."""
    word = status_word(device)
    outcome = torch.zeros(2, dtype=torch.int32, device=word.device)
    f = _fn("wait_probe", "jv_wait_probe", [c_longlong, c_int, c_void_p, c_void_p, c_void_p])
    with torch.cuda.device(word.device):
        _check(f(int(cycles), 1 if arrive else 0, word.data_ptr(), outcome.data_ptr(), _stream()), "wait_probe")
    done, spent = outcome.tolist()
    return done == 1, spent


# ------------------------------------------------------------------------ embedding
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """out[n, :] = table[ids[n], :] as float32; with `accumulate` the rows are added to `out`."""
    _cuda(table, "table"); _cuda(ids, "ids", torch.int32)
    n, (vocab, hidden) = ids.numel(), table.shape
    if accumulate and out is None:
        raise KernelError("embed_gather: accumulate needs `out`")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _cuda(out, "out", torch.float32)
    f = _fn("embed", "jv_embed_gather", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                         c_void_p])
    _check(f(table.data_ptr(), _code(table, "table"), ids.data_ptr(), out.data_ptr(), n, hidden, vocab,
             1 if accumulate else 0, _status_ptr(table.device), _stream()), "embed_gather")
    return out


# ----------------------------------------------------------------------------- norm
def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of rows of the float32 stream `h`, after adding `delta` (if given).

    Without `rows` every row is normalised and, when `delta` is given, `h` is updated
    in place with the sum.  With `rows` (int32) only those rows are produced and `h`
    stays as it is.
    """
    _cuda(h, "h", torch.float32); _cuda(weight, "weight")
    n_total, hidden = h.shape
    if weight.shape != (hidden,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, rows have {hidden} elements")
    delta, n_parts, part_stride = _delta_parts(delta, h)
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
    n_out = n_total if rows is None else rows.numel()
    y = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    f = _fn("norm", "jv_rmsnorm", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                   c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(h.data_ptr(), _ptr(delta), 0 if delta is None else _code(delta, "delta"), _ptr(rows),
             weight.data_ptr(), _code(weight, "weight"), y.data_ptr(), _code(y, "out"), n_out, n_total, hidden,
             float(eps), n_parts, part_stride, _status_ptr(h.device), _stream()), "rmsnorm")
    return y


def _delta_parts(delta, h: torch.Tensor):
    """(tensor, parts, elements between parts) for a `delta` that is a tensor, a PartialSum or None."""
    if delta is None:
        return None, 1, 0
    if isinstance(delta, (PickedRows, GatedDelta)):
        delta = delta.tensor()
    if isinstance(delta, PartialSum):
        parts = _cuda(delta.parts, "delta parts", torch.float32)
        if tuple(parts.shape[1:]) != tuple(h.shape):
            raise KernelError("delta and h differ in shape")
        return parts, parts.shape[0], parts.stride(0)
    _cuda(delta, "delta")
    if delta.shape != h.shape:
        raise KernelError("delta and h differ in shape")
    return delta, 1, 0


def residual_add(h: torch.Tensor, delta) -> torch.Tensor:
    """h += delta (a tensor, a PartialSum or a gated delta), the sum kept in float32."""
    _cuda(h, "h", torch.float32)
    if isinstance(delta, GatedDelta):
        gated_add_dyt(h, delta)
        return h
    delta, n_parts, part_stride = _delta_parts(delta, h)
    f = _fn("norm", "jv_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_int, c_longlong, c_void_p])
    _check(f(h.data_ptr(), delta.data_ptr(), _code(delta, "delta"), h.numel(), n_parts, part_stride, _stream()),
           "residual_add")
    return h


# ----------------------------------------------------------------------- activation
def swiglu(gate_up, block: int | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """silu(gate) * up for a packed [n, 2*inter] tensor: blocks of `block` gate columns, each followed
    by the up columns of the same indices (default: all gate columns first).  The input may be a
    PartialSum; the result then has `out_dtype`."""
    n_parts, part_stride = 1, 0
    if isinstance(gate_up, PartialSum):
        if out_dtype is None:
            raise KernelError("swiglu of a PartialSum needs out_dtype")
        gate_up = _cuda(gate_up.parts, "gate_up parts", torch.float32)
        n_parts, part_stride = gate_up.shape[0], gate_up.stride(0)
        n, two_i = gate_up.shape[1:]
        act_dtype = out_dtype
    else:
        _cuda(gate_up, "gate_up")
        n, two_i = gate_up.shape
        act_dtype = gate_up.dtype
    if two_i % 2:
        raise KernelError("packed gate|up needs an even number of columns")
    block = two_i // 2 if block is None else int(block)
    if block < 1 or (two_i // 2) % block:
        raise KernelError(f"gate|up block {block} does not divide {two_i // 2} columns")
    act = torch.empty((n, two_i // 2), dtype=act_dtype, device=gate_up.device)
    f = _fn("activation", "jv_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p])
    _check(f(gate_up.data_ptr(), act.data_ptr(), _code(act, "act"), n, two_i // 2, block, n_parts, part_stride, _stream()),
           "swiglu")
    return act


# --------------------------------------------------------- rope + q/k norm + kv write
def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor,
            inv_freq: torch.Tensor | None, q_norm_w, k_norm_w, eps: float, k_cache, v_cache,
            n_q_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Normalises and rotates the query and key heads of `qkv` in place and writes the new
    keys and values into the paged cache (see csrc/rope_kv.cu).  `inv_freq` None = no
    rotation.  `k_cache`/`v_cache` None = the layer writes no cache (queries only)."""
    _cuda(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(token_entry, "token_entry", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    n, width = qkv.shape
    heads = n_q_heads + (2 * n_kv_heads if k_cache is not None else 0)
    if width < heads * head_dim:
        raise KernelError(f"qkv has {width} columns, {heads} heads of {head_dim} need {heads * head_dim}")
    rot_dim = 0
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        rot_dim = 2 * inv_freq.numel()
    w_code = 0
    for w, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if w is not None:
            _cuda(w, nm)
            if w.shape != (head_dim,):
                raise KernelError(f"{nm} weight has shape {tuple(w.shape)}, head size is {head_dim}")
            w_code = _code(w, nm)
    if (q_norm_w is not None and k_norm_w is not None) and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q_norm and k_norm weights differ in dtype")
    page_size = num_pages = 1
    if k_cache is not None:
        _cuda(k_cache, "k_cache", qkv.dtype); _cuda(v_cache, "v_cache", qkv.dtype)
        if k_cache.shape != v_cache.shape or k_cache.shape[2:] != (n_kv_heads, head_dim):
            raise KernelError(f"cache shape {tuple(k_cache.shape)} does not fit {n_kv_heads} kv heads of {head_dim}")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
    f = _fn("rope_kv", "jv_rope_kv", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                      c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(qkv.data_ptr(), _code(qkv, "qkv"), qkv.stride(0), positions.data_ptr(), token_entry.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], _ptr(inv_freq), rot_dim, _ptr(q_norm_w), _ptr(k_norm_w),
             w_code, float(eps), _ptr(k_cache), _ptr(v_cache), n, n_q_heads, n_kv_heads, head_dim, page_size,
             num_pages, _status_ptr(qkv.device), _stream()), "rope_kv")


# ------------------------------------------------------------------------ attention
def mask_code(window: int | None = None, chunk: int | None = None) -> int:
    """The mask of an attention layer as the one number the kernels take (csrc/common.cuh, `first_visible`): n > 0, a
    query sees its own position and the n - 1 before it; n < 0, it sees the earlier positions of its own chunk of -n
    positions, chunks counted from position 0; 0, every earlier position."""
    if window and chunk:
        raise KernelError("a layer has a window or chunks, not both")
    return int(window) if window else -int(chunk) if chunk else 0


def attn_simt_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    g = n_q_heads // n_kv_heads
    return 16 // min(g, 16)


def attn_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
              n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
              split_size: int = 0, n_splits: int = 0, v_dim: int = 0, score_cap: float = 0.0, sigmoid: bool = False,
              bias: torch.Tensor | None = None, head_scale: torch.Tensor | None = None,
              dist_bias: torch.Tensor | None = None, sink: torch.Tensor | None = None) -> None:
    """Paged causal attention on CUDA cores (csrc/attn_simt.cu).  `work` is [n_work, 2] int32
    (entry, first token of the tile); with `n_splits` > 0 the work items are single tokens
    whose keys are split into `n_splits` ranges of `split_size` positions.  `v_dim` > 0: only that many
    leading elements of a value row are used and `out` has v_dim elements per head (a cache whose values are
    the leading part of its keys is passed as both caches).

    The value cache may have other heads and another row size than the key cache ([pages, page, value heads,
    value size]): key head g then reads value head g % value heads.  `score_cap` > 0 caps the scaled scores by
    cap * tanh(score / cap); `sigmoid` replaces the softmax by independent weights sigmoid(score + bias[query
    head]); `out` may be float32 whatever the type of q.  `head_scale` [query heads] multiplies the scaled scores of
    its head; `dist_bias` [query heads, distances] is added to the score of a key that lies so many positions back
    (the last column serves every larger distance); `sink` [query heads] adds exp(sink) once to the softmax's
    denominator."""
    n_dist = _score_extras("attn_simt", n_q_heads, head_scale, dist_bias, sink)
    for t, nm in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, q.dtype, contiguous=(nm != "q"))
    _cuda(out, "out", contiguous=False)
    if out.dtype not in (q.dtype, torch.float32) or out.stride(1) != 1:
        raise KernelError("attn_simt: out must have the type of q or float32, and unit column stride")
    if k_cache.dim() != 4 or v_cache.dim() != 4 or k_cache.shape[:2] != v_cache.shape[:2] or \
            k_cache.shape[2:] != (n_kv_heads, head_dim) or n_kv_heads % v_cache.shape[2]:
        raise KernelError(f"attn_simt: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit "
                          f"{n_kv_heads} key heads of {head_dim}")
    n_v_heads, v_row = v_cache.shape[2], v_cache.shape[3]
    v_dim = int(v_dim) or v_row
    if bias is not None:
        _cuda(bias, "bias", torch.float32)
        if bias.numel() != n_q_heads:
            raise KernelError("attn_simt: one bias per query head")
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    part_o = part_ml = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_q_heads * n_splits * v_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_q_heads * n_splits * 2, dtype=torch.float32, device=q.device)
    f = _fn("attn_simt", "jv_attn_simt_ex", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                             c_int, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), _code(q, "q"), _ptr(part_o), _ptr(part_ml),
             k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim,
             k_cache.shape[1], k_cache.shape[0], int(window), float(scale), int(split_size), int(n_splits), v_dim,
             n_v_heads, v_row, float(score_cap), 1 if sigmoid else 0, _ptr(bias), 1 if out.dtype != q.dtype else 0,
             _ptr(head_scale), _ptr(dist_bias), n_dist, _ptr(sink),
             _status_ptr(q.device), _stream()), "attn_simt", launches=2 if n_splits > 0 else 1)


def _score_extras(who: str, n_q_heads: int, head_scale, dist_bias, sink) -> int:
    """Checks the per-head score options of the attention kernels; returns the number of distances of the bias table."""
    for t, nm in ((head_scale, "head_scale"), (sink, "sink")):
        if t is not None:
            _cuda(t, nm, torch.float32)
            if t.numel() != n_q_heads:
                raise KernelError(f"{who}: {nm} holds one number per query head")
    if dist_bias is None:
        return 0
    _cuda(dist_bias, "dist_bias", torch.float32)
    if dist_bias.dim() != 2 or dist_bias.shape[0] != n_q_heads or dist_bias.shape[1] < 1:
        raise KernelError(f"{who}: dist_bias is [query heads, distances]")
    return dist_bias.shape[1]


GENERAL_MMA_MAX_KEY, GENERAL_MMA_MAX_VALUE = 256, 128


def attn_general_mma_supports(dtype: torch.dtype, key_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core kernel for keys and values of different sizes takes these (csrc/attn_general_mma.cu):
    bfloat16, sizes in steps of 16."""
    return (dtype == torch.bfloat16 and key_dim % 16 == 0 and value_dim % 16 == 0
            and 16 <= key_dim <= GENERAL_MMA_MAX_KEY and 16 <= value_dim <= GENERAL_MMA_MAX_VALUE)


def attn_general_mma_library(key_dim: int, value_dim: int) -> str:
    """The library of the kernel for this pair of sizes (compiled when first asked for)."""
    return f"attn_general_mma@{int(key_dim)}x{int(value_dim)}"


def attn_general_mma_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    return 64 // min(n_q_heads // n_kv_heads, 16)


def attn_general_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
                     n_work: int, n_q_heads: int, n_kv_heads: int, scale: float, split_size: int = 0, n_splits: int = 0,
                     score_cap: float = 0.0, sigmoid: bool = False, bias: torch.Tensor | None = None,
                     head_scale: torch.Tensor | None = None, dist_bias: torch.Tensor | None = None,
                     sink: torch.Tensor | None = None, window: int = 0) -> None:
    """Paged causal attention on the tensor cores with the options of `attn_simt`: the key size is the key
    cache's row, the value size and the value heads the value cache's; bfloat16 in, bfloat16 or float32 out.
    `window`: the mask as one number (`mask_code`)."""
    n_dist = _score_extras("attn_general_mma", n_q_heads, head_scale, dist_bias, sink)
    for t, nm in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    _cuda(out, "out", contiguous=False)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1:
        raise KernelError("attn_general_mma: out must be bfloat16 or float32 with unit column stride")
    if k_cache.dim() != 4 or v_cache.dim() != 4 or k_cache.shape[:2] != v_cache.shape[:2] or \
            k_cache.shape[2] != n_kv_heads or n_kv_heads % v_cache.shape[2]:
        raise KernelError(f"attn_general_mma: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit")
    key_dim, n_v_heads, value_dim = k_cache.shape[3], v_cache.shape[2], v_cache.shape[3]
    if bias is not None:
        _cuda(bias, "bias", torch.float32)
        if bias.numel() != n_q_heads:
            raise KernelError("attn_general_mma: one bias per query head")
    part_o = part_ml = counters = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_q_heads * n_splits * value_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_q_heads * n_splits * 2, dtype=torch.float32, device=q.device)
        counters = _split_counters(q.device, n_work * n_kv_heads * (-(-(n_q_heads // n_kv_heads) // 16)))
    f = _fn(attn_general_mma_library(key_dim, value_dim), "jv_attn_general_mma",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), 1 if out.dtype == torch.float32 else 0, _ptr(part_o),
             _ptr(part_ml), _ptr(counters), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads,
             n_kv_heads, n_v_heads, key_dim, value_dim, k_cache.shape[1], k_cache.shape[0], int(window), float(scale),
             float(score_cap), 1 if sigmoid else 0, _ptr(bias), _ptr(head_scale), _ptr(dist_bias), n_dist, _ptr(sink),
             int(split_size), int(n_splits), _status_ptr(q.device), _stream()), "attn_general_mma")


def attn_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, positions: torch.Tensor,
                 token_entry: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor | None,
                 q_norm_w, k_norm_w, eps: float, temp_coef: float, temp_every: int, k_cache, v_cache,
                 n_q_heads: int, n_k_heads: int, n_v_heads: int, key_dim: int, value_dim: int) -> None:
    """Prepares the queries, keys and values of a packed projection row for attention and writes the new keys and
    values into the paged cache (csrc/attn_prepare.cu): RMSNorm over a token's whole query (key) projection,
    a query temperature that grows with the position, rotation of the first `2 * len(inv_freq)` elements of every
    head.  Offsets are columns of `proj`; `v_off` < 0: the values are the keys as projected.  Queries go to
    `q_out` [n, n_q_heads * key_dim].  `k_cache`/`v_cache` None: queries only."""
    _cuda(proj, "proj", contiguous=False); _cuda(q_out, "q_out", proj.dtype)
    _cuda(positions, "positions", torch.int32); _cuda(token_entry, "token_entry", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    n, width = proj.shape
    if proj.stride(1) != 1 or q_out.shape != (n, n_q_heads * key_dim):
        raise KernelError("attn_prepare: proj needs unit column stride and q_out [n, query heads * key size]")
    writes = k_cache is not None
    ends = [q_off + n_q_heads * key_dim]
    if writes:
        ends += [k_off + n_k_heads * key_dim] + ([v_off + n_v_heads * value_dim] if v_off >= 0 else [])
    if min(q_off, k_off if writes else 0) < 0 or max(ends) > width:
        raise KernelError(f"attn_prepare: the heads do not fit a row of {width} columns")
    rot_dim = 0
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        rot_dim = 2 * inv_freq.numel()
    w_code = 0
    for w, nm, size in ((q_norm_w, "q_norm", n_q_heads * key_dim), (k_norm_w, "k_norm", n_k_heads * key_dim)):
        if w is not None:
            _cuda(w, nm)
            if w.numel() != size:
                raise KernelError(f"{nm} weight has {w.numel()} elements, the projection {size}")
            w_code = _code(w, nm)
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q_norm and k_norm weights differ in dtype")
    page_size = num_pages = 1
    if writes:
        _cuda(k_cache, "k_cache", proj.dtype); _cuda(v_cache, "v_cache", proj.dtype)
        if k_cache.shape[2:] != (n_k_heads, key_dim) or v_cache.shape[2:] != (n_v_heads, value_dim) or \
                k_cache.shape[:2] != v_cache.shape[:2]:
            raise KernelError(f"attn_prepare: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
    f = _fn("attn_prepare", "jv_attn_prepare",
            [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(proj.data_ptr(), _code(proj, "proj"), proj.stride(0), int(q_off), int(k_off), int(v_off), q_out.data_ptr(),
             positions.data_ptr(), token_entry.data_ptr(), block_table.data_ptr(), block_table.shape[1], _ptr(inv_freq),
             rot_dim, _ptr(q_norm_w), _ptr(k_norm_w), w_code, float(eps), float(temp_coef), int(temp_every),
             _ptr(k_cache), _ptr(v_cache), n, n_q_heads, n_k_heads, n_v_heads, key_dim, value_dim, page_size, num_pages,
             _status_ptr(proj.device), _stream()), "attn_prepare")


def attn_finish(a: torch.Tensor, out: torch.Tensor, heads: int, value_dim: int, maps: int = 1, lam: float = 0.0,
                unit_norm_eps: float | None = None, post: float = 1.0, gate: torch.Tensor | None = None) -> torch.Tensor:
    """Heads after attention, before the output projection (csrc/attn_finish.cu): with `maps` == 2 the difference
    a[:, h] - lam * a[:, heads + h] of two score maps on the same values; a weightless RMSNorm over each head
    (`unit_norm_eps`) times `post`; a sigmoid gate, one number per head (`gate` [n, heads]) or per element
    ([n, heads * value_dim]), which may be a column range of a wider tensor.  `a` [n, maps * heads * value_dim] is
    float32 or of the type of `out`; `out` [n, heads * value_dim] may be a column range of a wider tensor."""
    _cuda(a, "a"); _cuda(out, "out", contiguous=False)
    n = a.shape[0]
    if a.shape[1] != maps * heads * value_dim or out.shape != (n, heads * value_dim) or out.stride(1) != 1:
        raise KernelError("attn_finish: shapes do not fit")
    kind, g_stride = 0, 0
    if gate is not None:
        _cuda(gate, "gate", out.dtype, contiguous=False)
        if gate.stride(1) != 1 or gate.shape[0] != n or gate.shape[1] not in (heads, heads * value_dim):
            raise KernelError("attn_finish: the gate is [n, heads] or [n, heads * value size]")
        kind = 2 if gate.shape[1] == heads * value_dim and value_dim > 1 else 1
        g_stride = gate.stride(0)
    f = _fn("attn_finish", "jv_attn_finish", [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_int,
                                              c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_void_p])
    _check(f(a.data_ptr(), _code(a, "a"), out.data_ptr(), _code(out, "out"), out.stride(0), _ptr(gate), g_stride, kind,
             n, heads, value_dim, maps, float(lam), 0 if unit_norm_eps is None else 1, float(unit_norm_eps or 0.0),
             float(post), _stream()), "attn_finish")
    return out


UNARY_ACTIVATIONS = {"relu2": 0, "gelu": 1, "tanh": 2}       # relu(z)^2, the exact (erf) gelu, tanh


def unary_act(z: torch.Tensor, kind: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """act(z) element by element (csrc/activation.cu); `z` and `out` may be column ranges of wider tensors."""
    _cuda(z, "z", contiguous=False)
    n, cols = z.shape
    if out is None:
        out = torch.empty((n, cols), dtype=z.dtype, device=z.device)
    _cuda(out, "out", z.dtype, contiguous=False)
    if z.stride(1) != 1 or out.stride(1) != 1 or out.shape != z.shape:
        raise KernelError("unary_act: unit column strides and equal shapes")
    f = _fn("activation", "jv_unary_act", [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(z.data_ptr(), z.stride(0), out.data_ptr(), out.stride(0), _code(z, "z"), n, cols, UNARY_ACTIVATIONS[kind],
             _stream()), "unary_act")
    return out


MMA_HEAD_DIMS = (16, 32, 64, 128)      # head sizes the tensor-core attention kernels are instantiated for


def attn_mma_supports(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in MMA_HEAD_DIMS


def attn_mma_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    g = n_q_heads // n_kv_heads
    return 64 // min(g, 16)


def attn_latent_mma_supports(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """Whether the tensor-core attention over a latent cache takes rows of dk with values of dv
    (csrc/attn_latent_mma.cu): bfloat16, dk a multiple of 8 up to about 640, dv up to 512."""
    if dtype != torch.bfloat16 or dk % 8 or not 1 <= dv <= min(dk, 512):
        return False
    dkp = -(-dk // 16) * 16
    cols = (32 if dv <= 32 else 64 if dv <= 64 else 128 if dv <= 128 else 256) * (2 if dv > 256 else 1)
    return 2 * (64 * (dkp + 8) + 2 * 32 * (max(dkp, cols) + 8)) + (32768 if dv > 256 else 0) <= 220 * 1024


def attn_latent_mma_tokens_per_tile(n_heads: int) -> int:
    return 64 // min(n_heads, 64)


def attn_latent_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                    cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor, n_work: int, n_heads: int,
                    dk: int, dv: int, scale: float, split_size: int = 0, n_splits: int = 0, window: int = 0,
                    sink: torch.Tensor | None = None) -> None:
    """Paged causal attention with one key/value head whose key is the cache row [dk] and whose value is the row's
    first dv elements, on the tensor cores (csrc/attn_latent_mma.cu); `work` and the split arguments as for
    `attn_simt`, with `attn_latent_mma_tokens_per_tile` tokens per prompt tile; out has dv elements per head.
    `window`: the mask as one number (`mask_code`); `sink` [n_heads] float32: exp(sink) counts once in the denominator."""
    if sink is not None:
        _cuda(sink, "sink", torch.float32)
        if sink.numel() != n_heads:
            raise KernelError("attn_latent_mma: a sink per head")
    for t, nm in ((q, "q"), (out, "out"), (cache, "cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    if cache.shape[2:] != (1, dk):
        raise KernelError(f"cache shape {tuple(cache.shape)} does not fit rows of {dk}")
    part_o = part_ml = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_heads * n_splits * dv, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_heads * n_splits * 2, dtype=torch.float32, device=q.device)
    f = _fn("attn_latent_mma", "jv_attn_latent_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                      c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), _ptr(part_o), _ptr(part_ml), cache.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(),
             n_work, n_heads, dk, dv, cache.shape[1], cache.shape[0], float(scale), int(window), _ptr(sink),
             int(split_size), int(n_splits), _status_ptr(q.device), _stream()), "attn_latent_mma", launches=2 if n_splits > 0 else 1)


_counters: dict[int, torch.Tensor] = {}
_counters_outgrown: list = []     # smaller buffers that a captured graph may still point at: never freed


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed arrival counters for the split decode attention: one buffer per device, kept for
    the life of the process (the kernel leaves the counters zero; launches on one stream follow
    one another, so they can share it)."""
    idx = torch.device(device).index
    idx = torch.cuda.current_device() if idx is None else idx
    buf = _counters.get(idx)
    if buf is None or buf.numel() < n:
        if buf is not None:
            _counters_outgrown.append(buf)
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _counters[idx] = buf
    return buf


def attn_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
             n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
             split_size: int = 0, n_splits: int = 0) -> None:
    """Paged causal attention for bfloat16 on the tensor cores (csrc/attn_mma.cu); arguments as
    for `attn_simt`, with `attn_mma_tokens_per_tile` tokens per prompt tile."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    part_o = part_ml = counters = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_q_heads * n_splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_q_heads * n_splits * 2, dtype=torch.float32, device=q.device)
        counters = _split_counters(q.device, n_work * n_kv_heads * (-(-(n_q_heads // n_kv_heads) // 16)))
    f = _fn("attn_mma", "jv_attn_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), _ptr(part_o), _ptr(part_ml), _ptr(counters),
             k_cache.data_ptr(),
             v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(),
             start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim, k_cache.shape[1],
             k_cache.shape[0], int(window), float(scale), int(split_size), int(n_splits),
             _status_ptr(q.device), _stream()), "attn_mma")


def attn_tcgen05_supports(dtype: torch.dtype, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int,
                          window: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes the case (csrc/attn_tcgen05.cu)."""
    g = n_q_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and n_q_heads % n_kv_heads == 0
            and 1 <= g <= 16 and page_size in (8, 16, 32, 64, 128))      # any mask (`window`) is taken


def attn_tcgen05_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    return 128 // (n_q_heads // n_kv_heads)


def attn_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
                 n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, sigmoid: bool = False,
                 bias: torch.Tensor | None = None, head_scale: torch.Tensor | None = None,
                 dist_bias: torch.Tensor | None = None, sink: torch.Tensor | None = None, window: int = 0) -> None:
    """Paged causal attention of prompt portions on tcgen05 tensor cores with scores and output in tensor
    memory (csrc/attn_tcgen05.cu); `work` lists 128-row tiles of `attn_tcgen05_tokens_per_tile` tokens.  With
    `sigmoid` the weight of a visible key is sigmoid(score * scale + bias[query head]) instead of a softmax;
    `head_scale`, `dist_bias` and `sink` as for `attn_simt` (softmax only); `window`: the mask as one number
    (`mask_code`)."""
    n_dist = _score_extras("attn_tcgen05", n_q_heads, head_scale, dist_bias, sink)
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm not in ("q", "out")))     # q and out may be some heads of wider rows
    if out.stride(1) != 1 or q.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    if bias is not None:
        _cuda(bias, "bias", torch.float32)
        if bias.numel() != n_q_heads:
            raise KernelError("attn_tcgen05: one bias per query head")
    f = _fn("attn_tcgen05", "jv_attn_tcgen05_ex", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                   c_int, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(),
             n_work, n_q_heads, n_kv_heads, head_dim, k_cache.shape[1], k_cache.shape[0], float(scale),
             1 if sigmoid else 0, _ptr(bias), _ptr(head_scale), _ptr(dist_bias), n_dist, _ptr(sink), int(window),
             _status_ptr(q.device), _stream()), "attn_tcgen05")


DECODE_TCGEN05_MAX_REQUESTS = 512


def attn_decode_tcgen05_supports(dtype: torch.dtype, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int,
                                 window: int, n_requests: int = 1) -> bool:
    """Whether the tcgen05 decode-attention kernel takes the case (csrc/attn_decode_tcgen05.cu)."""
    return (dtype == torch.bfloat16 and head_dim == 128 and not window and n_kv_heads > 0
            and n_q_heads % n_kv_heads == 0 and n_q_heads // n_kv_heads <= 16
            and n_requests <= DECODE_TCGEN05_MAX_REQUESTS and page_size in (8, 16, 32, 64, 128))


_sm_count: dict = {}


def multiprocessors(device) -> int:
    """Multiprocessors of the device (what dispatch rules are scaled by)."""
    return _multiprocessors(device)


def _multiprocessors(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def attn_decode_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
                        work: torch.Tensor, n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                        scale: float, prepare: tuple | None = None) -> None:
    """Decode attention (single tokens) with the keys of a tile as tensor-core rows and scores and output in
    tensor memory; one persistent launch shares the key tiles of all requests evenly among the
    multiprocessors (csrc/attn_decode_tcgen05.cu).  `work`, `cu_seqlens`, `start_pos` as for `attn_mma`.

    `prepare` = (inv_freq or None, q_norm_weight or None, k_norm_weight or None, eps): `q` is then the product
    q|k|v as it comes, and the kernel does what `rope_kv` does for these tokens itself (per-head norm,
    rotation at position start_pos, write of the new key and value into the caches)."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm not in ("q", "out")))     # q and out may be some heads of wider rows
    if out.stride(1) != 1 or q.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    inv_freq = q_w = k_w = None
    eps, w_f32 = 0.0, 0
    if prepare is not None:
        inv_freq, q_w, k_w, eps = prepare
        if inv_freq is not None:
            _cuda(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() != head_dim // 2:
                raise KernelError("the kernel rotates whole heads only")
        if (q_w is None) != (k_w is None):
            raise KernelError("norm weights for queries and keys come together")
        if q_w is not None:
            _cuda(q_w, "q_norm_weight"); _cuda(k_w, "k_norm_weight")
            if q_w.dtype != k_w.dtype or q_w.numel() != head_dim or k_w.numel() != head_dim:
                raise KernelError("norm weights must have one dtype and head_dim elements")
            w_f32 = 1 if q_w.dtype == torch.float32 else 0
            _code(q_w, "q_norm_weight")
    n_blocks = _multiprocessors(q.device)
    slots = n_work * n_kv_heads + n_blocks
    g = n_q_heads // max(n_kv_heads, 1)
    part_o = torch.empty(slots * g * head_dim, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(slots * g * 2, dtype=torch.float32, device=q.device)
    counters = _split_counters(q.device, n_work * n_kv_heads)
    f = _fn("attn_decode_tcgen05", "jv_attn_decode_tcgen05",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.stride(0), part_o.data_ptr(), part_ml.data_ptr(),
             counters.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim,
             k_cache.shape[1], k_cache.shape[0], float(scale), n_blocks, 0 if prepare is None else 1, _ptr(inv_freq),
             _ptr(q_w), _ptr(k_w), w_f32, float(eps), _status_ptr(q.device), _stream()),
           "attn_decode_tcgen05")


# --------------------------------------------------------------------------- linear
def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, accumulated in float32 on CUDA cores."""
    _cuda(x, "x", contiguous=False); _cuda(weight, "weight")
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1:
        raise KernelError(f"gemm shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("gemm_simt", "jv_gemm_tn_simt", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_void_p])
    _check(f(x.data_ptr(), _code(x, "x"), x.stride(0), weight.data_ptr(), _code(weight, "weight"), weight.stride(0),
             y.data_ptr(), _code(y, "out"), y.stride(0), m, n, k, _stream()), "gemm_simt")
    return y


SKINNY_MAX_ROWS = 16      # rows the mma.sync kernel takes (in a replayed decode step it beats the library up to there)


_skinny_plans: dict = {}      # (device, N, K) -> parts of k per strip


def linear_skinny_splits(device, n: int, k: int) -> int:
    """Into how many parts of k the kernel would best cut the strips of an [n, k] weight on this device
    (1: not at all): few strips, or strips that load the multiprocessors unevenly, are cut."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n, k)
    plan = _skinny_plans.get(key)
    if plan is None:
        f = _build.load("linear_skinny").jv_linear_skinny_plan
        f.argtypes = [c_int, c_int]
        f.restype = c_int
        with torch.cuda.device(key[0]):
            plan = _skinny_plans[key] = int(f(n, k))
    return plan


# Where the caller wants one tensor, the kernel's strips are not cut, and a number of strips just above a multiple of
# the resident blocks leaves most of them idle for a second round: below this evenness (the useful share of the busiest
# block's time, csrc/linear_skinny.cu) the library's product is taken instead.  7,168 x 5,120 (448 strips for 444
# blocks): 0.50 and 20.4 against 14.1 us; 6,144 x 4,096: 1; 10,240 x 5,120: 0.72 and 22.6 against 21.8 us alone,
# where starting under the kernel before still favours the kernel.
SKINNY_MIN_EVENNESS = 0.6
_skinny_fill: dict = {}


def linear_skinny_evenness(device, n: int) -> float:
    """How evenly the uncut 16-row strips of a weight of n rows fill the rounds of this device's resident blocks
    (1: every strip has a block of its own, or the rounds are full)."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n)
    fill = _skinny_fill.get(key)
    if fill is None:
        f = _build.load("linear_skinny").jv_linear_skinny_fill
        f.argtypes, f.restype = [c_int], c_int
        with torch.cuda.device(key[0]):
            fill = _skinny_fill[key] = f(n) / 1000.0
    return fill


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, parts_ok: bool = False):
    """x [M <= 16, K] times weight [N, K] transposed, bfloat16 operands, 32-bit accumulation
    (csrc/linear_skinny.cu); the result is bfloat16 or float32, or with `parts_ok`, where the kernel cuts k
    for an even load, a PartialSum for a reader that adds the parts."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"linear shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    splits = linear_skinny_splits(x.device, n, k) if parts_ok else 1
    if splits > 1:
        parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        y = None
    else:
        parts = None
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("linear_skinny", "jv_linear_skinny", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(y), DTYPE_CODE[out_dtype],
             n if y is None else y.stride(0), m, n, k, _ptr(parts), splits, _stream()), "linear_skinny")
    return y if parts is None else PartialSum(parts)


STREAM_MAX_ROWS = 128
# up to this many rows the dispatcher takes the tcgen05 product of this package, beyond that the library's (which
# shares x between two multiprocessors)
STREAM_BEST_ROWS = 64
_stream_plans: dict = {}


def linear_stream_splits(device, n: int, k: int) -> int:
    """Into how many parts of k the product for 17 to 128 rows (csrc/linear_stream.cu) would best cut the
    128-row strips of an [n, k] weight on this device (1: not at all)."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n, k)
    plan = _stream_plans.get(key)
    if plan is None:
        f = _build.load("linear_stream").jv_linear_stream_plan
        f.argtypes = [c_int, c_int]
        f.restype = c_int
        with torch.cuda.device(key[0]):
            plan = _stream_plans[key] = int(f(n, k))
    return plan


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, parts_ok: bool = False):
    """x [M <= 128, K] times weight [N, K] transposed on tcgen05 with the weight as the 128-row operand and the
    batch as the narrow one (csrc/linear_stream.cu): bfloat16 operands, 32-bit accumulation; the result is
    bfloat16 or float32, or with `parts_ok`, where the kernel cuts k for an even load, a PartialSum."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"linear shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    splits = linear_stream_splits(x.device, n, k) if parts_ok else 1
    if splits > 1:
        parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        y = None
    else:
        parts = None
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("linear_stream", "jv_linear_stream", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(y), DTYPE_CODE[out_dtype],
             n if y is None else y.stride(0), m, n, k, _ptr(parts), splits, _status_ptr(x.device), _stream()),
           "linear_stream")
    return y if parts is None else PartialSum(parts)


def _stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dim() == 2 and 0 < x.shape[0] <= STREAM_MAX_ROWS and x.stride(1) == 1 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and x.dtype == torch.bfloat16)


GEMM_EPILOGUES = {"bf16": 0, "f32": 1, "swiglu": 2, "gelu": 3}


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "bf16") -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed on tcgen05 tensor cores with the accumulator in
    tensor memory (csrc/gemm_tcgen05.cu).  epilogue "bf16" / "f32": the product in that type;
    "swiglu": silu(gate) * up as [M, N/2] bfloat16, for a weight whose every 256 rows are 128 gate rows
    followed by the 128 up rows of the same indices."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"gemm shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    code = GEMM_EPILOGUES[epilogue]
    if epilogue == "swiglu":
        y = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
    else:
        y = torch.empty((m, n), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=x.device)
    f = _fn("gemm_tcgen05", "jv_gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), y.data_ptr(), y.stride(0), m, n, k, code,
             _status_ptr(x.device), _stream()), "gemm_tcgen05")
    return y


_sm_counts: dict = {}


_strips_fill: dict = {}


def _strips_fill_the_device(device, n: int) -> bool:
    """Whether the 128-row strips of a weight of n rows, uncut, keep the multiprocessors busy (0.85 of them over
    the rounds it takes): the tcgen05 product for larger batches takes a weight whole only then."""
    idx = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    fills = _strips_fill.get((idx, n))
    if fills is None:
        sms = _sm_counts.get(idx)
        if sms is None:
            sms = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
        strips = -(-n // 128)
        fills = _strips_fill[(idx, n)] = strips >= 0.85 * sms * -(-strips // sms)
    return fills


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.stride(1) == 1)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None, parts_ok: bool = False):
    """y = x @ weight.T.  With `parts_ok` the result may be a PartialSum (the caller hands it to `rmsnorm`,
    `residual_add` or `swiglu`, which add its parts as they read them).

    float32 weights: the CUDA-core product of this package in true 32-bit (16-bit activations are read as they
    are and widened inside).  bfloat16 weights and activations: up to STREAM_BEST_ROWS rows (decoding) the
    weight-streaming product on tcgen05 (csrc/linear_stream.cu), which cuts the k of a weight with few strips into
    parts; where the reader wants one tensor and the strips are few, the mma.sync product (csrc/linear_skinny.cu, up
    to SKINNY_MAX_ROWS rows), whose strips are 16 rows; else (prompts) cuBLAS through torch.mm.  All
    accumulate in 32-bit and give the result in `out_dtype` (bfloat16 by default, float32 for logits)."""
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32 or x.dtype == torch.float32:
        return gemm_simt(x, weight, out_dtype)
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16)
    if _stream_ok(x, weight) and x.shape[0] <= STREAM_BEST_ROWS and out_dtype in (torch.bfloat16, torch.float32) and \
            (parts_ok or _strips_fill_the_device(x.device, weight.shape[0])):
        return linear_stream(x, weight, out_dtype, parts_ok)
    if _skinny_ok(x, weight) and (parts_ok or linear_skinny_evenness(x.device, weight.shape[0]) >= SKINNY_MIN_EVENNESS):
        return linear_skinny(x, weight, out_dtype, parts_ok)
    if out_dtype == torch.bfloat16:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=out_dtype)


# ------------------------------------------------- layers that norm a branch's output
def branch_norm_add(h: torch.Tensor, branch, weight: torch.Tensor, eps: float, mult: float,
                    x_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """h += mult * rmsnorm(branch) * weight, in 32-bit and in place (csrc/branch_norm.cu); returns h rounded to
    `x_dtype` (what the next branch reads), or None if no `x_dtype` is given.  `branch` is a tensor [n, hidden], a
    PartialSum or a PickedRows; the latter two are added up as they are read."""
    _cuda(h, "h", torch.float32); _cuda(weight, "weight")
    pick = coef = None
    if isinstance(branch, PickedRows):
        branch, pick, coef = branch.rows, branch.pick, branch.coef
    n, hidden = h.shape
    if weight.shape != (hidden,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, rows have {hidden} elements")
    parts, part_stride, y_rows = 1, 0, n
    if pick is not None:
        _cuda(pick, "pick", torch.int32); _cuda(coef, "coef", torch.float32); _cuda(branch, "branch")
        if pick.shape != coef.shape or pick.shape[0] != n or branch.shape[1] != hidden:
            raise KernelError("pick, coef and branch do not fit the stream")
        parts, y_rows, y = pick.shape[1], branch.shape[0], branch
    else:
        y, parts, part_stride = _delta_parts(branch, h)
    x = torch.empty((n, hidden), dtype=x_dtype, device=h.device) if x_dtype is not None else None
    f = _fn("branch_norm", "jv_branch_norm_add", [c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                                  c_void_p, c_void_p])
    _check(f(h.data_ptr(), y.data_ptr(), _code(y, "branch"), part_stride, parts, _ptr(pick), _ptr(coef), y_rows,
             weight.data_ptr(), _code(weight, "weight"), _ptr(x), 0 if x is None else _code(x, "x"), n, hidden,
             float(eps), float(mult), _status_ptr(h.device), _stream()), "branch_norm_add")
    return x


def cast_rows(h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream rounded to `dtype` (the stream itself for float32)."""
    _cuda(h, "h", torch.float32)
    if dtype == torch.float32:
        return h
    x = torch.empty_like(h, dtype=dtype)
    f = _fn("branch_norm", "jv_cast_rows", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(h.data_ptr(), x.data_ptr(), _code(x, "x"), h.numel(), _stream()), "cast_rows")
    return x


# ------------------------------------------------------------------ latent attention
def latent_prepare(row: torch.Tensor, q_off: int, kv_off: int, q_latent: torch.Tensor | None, q_out: torch.Tensor,
                   positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor,
                   inv_freq: torch.Tensor | None, norm_w: torch.Tensor | None, eps: float, cache: torch.Tensor | None,
                   heads: int, plain_dim: int, rot_dim: int, latent_dim: int, kv_row: torch.Tensor | None = None,
                   interleaved: bool = False) -> None:
    """Writes a token's cache row [normed latent | rotated key part] and puts its query row together as
    [q_latent | rotated query part] per head (csrc/latent_prepare.cu).  `row`: the product rows
    [queries | down-projection]; `kv_off` < 0 or `cache` None: queries only.  `q_latent` [heads, n, latent_dim]
    is copied into `q_out` if given (else it is there already).  `kv_row`: the rows that hold the down-projection at
    `kv_off`, where the queries come from a product of their own.  `interleaved`: the rotation pairs element 2i with
    2i + 1 instead of i with i + rot_dim / 2."""
    _cuda(row, "row", contiguous=False); _cuda(q_out, "q_out", row.dtype)
    if kv_row is not None:
        _cuda(kv_row, "kv_row", row.dtype, contiguous=False)
        if kv_row.shape[0] != row.shape[0] or kv_row.stride(1) != 1:
            raise KernelError("kv_row has a row per token")
    _cuda(positions, "positions", torch.int32); _cuda(token_entry, "token_entry", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    n = row.shape[0]
    dk = latent_dim + rot_dim
    if q_out.shape != (n, heads * dk):
        raise KernelError(f"q_out has shape {tuple(q_out.shape)}, expected {(n, heads * dk)}")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if 2 * inv_freq.numel() != rot_dim:
            raise KernelError("the rotation table does not fit the rotated part")
    if q_latent is not None:
        _cuda(q_latent, "q_latent", row.dtype)
        if q_latent.shape != (heads, n, latent_dim):
            raise KernelError("q_latent must be [heads, n, latent_dim]")
    writes = cache is not None and kv_off >= 0
    page_size = num_pages = 1
    if writes:
        _cuda(cache, "cache", row.dtype); _cuda(norm_w, "latent norm weight")
        if cache.shape[2:] != (1, dk) or norm_w.shape != (latent_dim,):
            raise KernelError(f"cache shape {tuple(cache.shape)} does not fit rows of {dk}")
        if (row if kv_row is None else kv_row).shape[1] < kv_off + dk:
            raise KernelError("the product row is too short for the down-projection")
        num_pages, page_size = cache.shape[0], cache.shape[1]
    f = _fn("latent_prepare", "jv_latent_prepare",
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_int, c_int, c_void_p, c_void_p])
    _check(f(row.data_ptr(), _code(row, "row"), row.stride(0), q_off, kv_off if writes else -1, _ptr(q_latent),
             q_out.data_ptr(), q_out.stride(0), positions.data_ptr(), token_entry.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], _ptr(inv_freq), _ptr(norm_w) if writes else 0,
             _code(norm_w, "norm") if writes else 0, float(eps), _ptr(cache) if writes else 0, n, heads, plain_dim,
             rot_dim, latent_dim, page_size, num_pages, _ptr(kv_row), 0 if kv_row is None else kv_row.stride(0),
             1 if interleaved else 0, _status_ptr(row.device), _stream()), "latent_prepare")


def gate_heads(o: torch.Tensor, gate: torch.Tensor | None) -> torch.Tensor:
    """out[t, h*dv + d] = o[h, t, d] * sigmoid(gate[t, h*dv + d]) (no gate: the re-ordering alone);
    `gate` may be a column slice of a wider tensor."""
    _cuda(o, "o")
    heads, n, dv = o.shape
    g_stride = 0
    if gate is not None:
        _cuda(gate, "gate", o.dtype, contiguous=False)
        if gate.shape != (n, heads * dv) or gate.stride(1) != 1:
            raise KernelError("gate must be [n, heads * dv] with unit column stride")
        g_stride = gate.stride(0)
    out = torch.empty((n, heads * dv), dtype=o.dtype, device=o.device)
    f = _fn("latent_prepare", "jv_gate_heads", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(o.data_ptr(), _ptr(gate), g_stride, out.data_ptr(), _code(o, "o"), n, heads, dv, _stream()), "gate_heads")
    return out


def bmm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One product per head: out[h] = a[h] @ w[h].T, a [heads, n, k] (any strides with unit inner stride),
    w [heads, m, k] contiguous, out [heads, n, m] (made contiguous if not given; given, any strides with unit
    inner stride).  float32 operands: the CUDA-core product of this package, k ascending (csrc/gemm_simt.cu);
    bfloat16: the library's batched product (as the prompt products of this package are the library's)."""
    _cuda(a, "a", contiguous=False); _cuda(w, "w", a.dtype)
    heads, n, k = a.shape
    m = w.shape[1]
    if w.shape != (heads, m, k) or a.stride(2) != 1:
        raise KernelError(f"batched product shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not fit")
    if a.dtype != torch.float32:
        if out is None:
            return torch.bmm(a, w.transpose(1, 2))
        out.copy_(torch.bmm(a, w.transpose(1, 2)))
        return out
    if out is None:
        out = torch.empty((heads, n, m), dtype=a.dtype, device=a.device)
    _cuda(out, "out", a.dtype, contiguous=False)
    if out.shape != (heads, n, m) or out.stride(2) != 1:
        raise KernelError("out does not fit the batched product")
    f = _fn("gemm_simt", "jv_gemm_tn_simt_batched", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_longlong,
                                                    c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                                    c_void_p])
    _check(f(a.data_ptr(), _code(a, "a"), a.stride(1), a.stride(0), w.data_ptr(), _code(w, "w"), w.stride(1), w.stride(0),
             out.data_ptr(), _code(out, "out"), out.stride(1), out.stride(0), n, m, k, heads, _stream()), "bmm_heads")
    return out


# ------------------------------------------------------------------- routed experts
ROUTER_SCORINGS = {"softmax": 0, "sigmoid": 1}
GROUP_SCORES = {"max": 0, "top2_sum": 1}


def moe_route(logits: torch.Tensor, top: int, groups: int, keep: int, renorm: bool, scoring: str = "softmax",
              group_score: str = "max", renorm_eps: float = 0.0, weight_scale: float = 1.0):
    """(ids [n, top] int32, weights [n, top] float32) from the router logits [n, experts] float32: softmax over all
    experts or a sigmoid of each, group-limited choice of the `top` largest, largest first (csrc/moe_route.cu); a
    group scores as its best expert or as the sum of its two best; the chosen scores are divided by their sum
    (+ `renorm_eps`) if `renorm`, and multiplied by `weight_scale`."""
    _cuda(logits, "router logits", torch.float32, contiguous=False)
    n, experts = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("router logits need unit column stride")
    ids = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    f = _fn("moe_route", "jv_moe_route", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                          c_float, c_void_p, c_void_p, c_void_p])
    _check(f(logits.data_ptr(), logits.stride(0), n, experts, top, groups, keep, 1 if renorm else 0,
             ROUTER_SCORINGS[scoring], GROUP_SCORES[group_score], float(renorm_eps), float(weight_scale), ids.data_ptr(),
             weights.data_ptr(), _stream()), "moe_route")
    return ids, weights


def moe_align(ids: torch.Tensor, experts: int, tile: int):
    """The (token, choice) pairs in the order of their experts, each expert's run padded to `tile` rows:
    (sorted_token [max_tiles * tile] (-1: padding), pos_of [n, top], tile_expert [max_tiles] (-1: unused), and
    a one-element tensor: how many leading tiles are in use)."""
    _cuda(ids, "ids", torch.int32)
    n, top = ids.shape
    pairs = n * top
    max_tiles = -(-(pairs + experts * (tile - 1)) // tile)
    sorted_token = torch.empty(max_tiles * tile, dtype=torch.int32, device=ids.device)
    pos_of = torch.empty((n, top), dtype=torch.int32, device=ids.device)
    tile_expert = torch.empty(max_tiles + 1, dtype=torch.int32, device=ids.device)
    f = _fn("moe_route", "jv_moe_align", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p])
    _check(f(ids.data_ptr(), pairs, top, experts, tile, max_tiles, sorted_token.data_ptr(), pos_of.data_ptr(),
             tile_expert.data_ptr(), _status_ptr(ids.device), _stream()), "moe_align")
    return sorted_token, pos_of, tile_expert[:max_tiles], tile_expert[max_tiles:]


MOE_ACTS = {None: 0, "gelu": 1}


def moe_gemm_simt_tile() -> int:
    f = _build.load("moe_gemm_simt").jv_moe_gemm_simt_tile
    f.argtypes, f.restype = [], c_int
    return int(f())


def moe_gemm_simt(a: torch.Tensor, gather: torch.Tensor | None, w: torch.Tensor, tile_expert: torch.Tensor,
                  out_dtype: torch.dtype, act: str | None = None) -> torch.Tensor:
    """Grouped product on CUDA cores (csrc/moe_gemm_simt.cu): row pos of the result, in a tile of expert e, is
    act(a[gather[pos]] @ w[e].T) (gather None: a[pos]); w [experts, N, K]; rows of padding are left unwritten."""
    _cuda(a, "a"); _cuda(w, "w"); _cuda(tile_expert, "tile_expert", torch.int32)
    tile = moe_gemm_simt_tile()
    max_tiles = tile_expert.numel()
    experts, n_out, k = w.shape
    if a.shape[1] != k:
        raise KernelError("grouped product: inner sizes differ")
    if gather is not None:
        _cuda(gather, "gather", torch.int32)
        if gather.numel() != max_tiles * tile:
            raise KernelError("gather does not fit the tiles")
    elif a.shape[0] != max_tiles * tile:
        raise KernelError("rows do not fit the tiles")
    out = torch.empty((max_tiles * tile, n_out), dtype=out_dtype, device=a.device)
    f = _fn("moe_gemm_simt", "jv_moe_gemm_simt", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_longlong, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                  c_void_p])
    _check(f(a.data_ptr(), _code(a, "a"), a.stride(0), _ptr(gather), a.shape[0], w.data_ptr(), _code(w, "w"), w.stride(0),
             w.stride(1), tile_expert.data_ptr(), max_tiles, out.data_ptr(), _code(out, "out"), out.stride(0), n_out, k,
             MOE_ACTS[act], _status_ptr(a.device), _stream()), "moe_gemm_simt")
    return out


def moe_gather_rows(x: torch.Tensor, pos_of: torch.Tensor, out_rows: int) -> torch.Tensor:
    """The rows of `x` [n, width] in the order of their experts: out[pos_of[t, k]] = x[t]; rows of padding are
    left as they are (csrc/moe_route.cu)."""
    _cuda(x, "x", contiguous=False); _cuda(pos_of, "pos_of", torch.int32)
    n, width = x.shape
    if pos_of.shape[0] != n or x.stride(1) != 1:
        raise KernelError("pos_of does not fit the rows")
    out = torch.empty((out_rows, width), dtype=x.dtype, device=x.device)
    f = _fn("moe_route", "jv_moe_gather_rows", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                                c_void_p])
    _check(f(x.data_ptr(), _code(x, "x"), x.stride(0), pos_of.data_ptr(), pos_of.numel(), pos_of.shape[1], out.data_ptr(),
             out_rows, width, _stream()), "moe_gather_rows")
    return out


MOE_TCGEN05_TILE = 128


def moe_gemm_tcgen05_supports(dtype: torch.dtype, w: torch.Tensor) -> bool:
    """Whether the grouped tcgen05 product takes these expert matrices [experts, N, K] (csrc/gemm_tcgen05.cu)."""
    return (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 3 and w.is_contiguous()
            and w.shape[2] % 8 == 0 and w.shape[2] >= 8 and w.data_ptr() % 16 == 0)


def moe_gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, act: str | None = None,
                     used_tiles: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped product on tcgen05 (csrc/gemm_tcgen05.cu): row pos of the result, in a 128-row tile of expert e, is
    act(a[pos] @ w[e].T); a [max_tiles * 128, K] bfloat16 in the order of the experts, w [experts, N, K];
    `used_tiles`: one int32 on the device, how many leading tiles have an expert."""
    _cuda(a, "a", torch.bfloat16); _cuda(w, "w", torch.bfloat16); _cuda(tile_expert, "tile_expert", torch.int32)
    if used_tiles is not None:
        _cuda(used_tiles, "used_tiles", torch.int32)
    max_tiles = tile_expert.numel()
    experts, n_out, k = w.shape
    if a.shape != (max_tiles * MOE_TCGEN05_TILE, k):
        raise KernelError("grouped product: rows do not fit the tiles")
    out = torch.empty((a.shape[0], n_out), dtype=torch.bfloat16, device=a.device)
    f = _fn("gemm_tcgen05", "jv_moe_gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                                    c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(1), experts, tile_expert.data_ptr(), max_tiles,
             _ptr(used_tiles), out.data_ptr(), out.stride(0), n_out, k, GEMM_EPILOGUES["gelu" if act == "gelu" else "bf16"],
             _status_ptr(a.device), _stream()), "moe_gemm_tcgen05")
    return out


# ---------------------------------------------------------------- per-layer token input
def token_gate(z: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, offset: int,
               out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """g[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], offset + j] in `out_dtype` (z's by default)
    (csrc/token_input.cu)."""
    _cuda(z, "z"); _cuda(tokens, "tokens", torch.int32); _cuda(table, "table")
    n, dim = z.shape
    vocab, width = table.shape
    if offset < 0 or offset + dim > width or tokens.numel() != n:
        raise KernelError("token table does not fit")
    g = torch.empty_like(z, dtype=out_dtype or z.dtype)
    f = _fn("token_input", "jv_token_gate", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                             c_int, c_int, c_void_p, c_void_p])
    _check(f(z.data_ptr(), _code(z, "z"), _code(g, "g"), tokens.data_ptr(), table.data_ptr(), _code(table, "table"), width, offset,
             vocab, g.data_ptr(), n, dim, _status_ptr(z.device), _stream()), "token_gate")
    return g


# ------------------------------------------------- clamped gate, logit cap (csrc/activation.cu)
def glu_clamped(gu: torch.Tensor, limit: float, slope: float = 1.702) -> torch.Tensor:
    """act = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), from rows
    [gate | up] (32-bit arithmetic)."""
    _cuda(gu, "gate|up")
    n, two = gu.shape
    if two % 2:
        raise KernelError("glu_clamped: rows hold gate and up columns of equal number")
    act = torch.empty((n, two // 2), dtype=gu.dtype, device=gu.device)
    f = _fn("activation", "jv_glu_clamped", [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(f(gu.data_ptr(), act.data_ptr(), _code(gu, "gate|up"), n, two // 2, float(limit), float(slope), _stream()),
           "glu_clamped")
    return act


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), in place on float32 values."""
    _cuda(x, "x", torch.float32)
    f = _fn("activation", "jv_softcap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(x.data_ptr(), x.numel(), float(cap), _stream()), "softcap")
    return x


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x <- x * factor, in place on float32 values."""
    _cuda(x, "x", torch.float32)
    f = _fn("activation", "jv_scale", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(x.data_ptr(), x.numel(), float(factor), _stream()), "scale")
    return x


# ------------------------------------------ dynamic-tanh norm and gated residual (csrc/dyt.cu)
class GatedDelta:
    """A branch output that enters the stream through a gate: the sum is h += sigmoid(z + bias) * y, element by
    element, in 32-bit.  `y` [n, hidden] (compute type or float32), `z` [n, hidden] (possibly a column range of a
    wider tensor), `bias` [hidden].  `gated_add_dyt` adds it as it forms the next norm; `residual_add` and
    `tensor()` serve any other reader."""

    def __init__(self, y: torch.Tensor, z: torch.Tensor, bias: torch.Tensor):
        self.y, self.z, self.bias = y, z, bias

    @property
    def shape(self):
        return self.y.shape

    @property
    def device(self):
        return self.y.device

    def tensor(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.zeros(tuple(self.shape), dtype=torch.float32, device=self.device)
        gated_add_dyt(out, self)
        return out if dtype == torch.float32 else out.to(dtype)


def gated_add_dyt(h: torch.Tensor, delta=None, alpha: float = 0.0, weight: torch.Tensor | None = None,
                  bias: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                  rows: torch.Tensor | None = None):
    """h += delta (a tensor, a `GatedDelta`, or anything with `.tensor()`), then, with `weight`, the dynamic-tanh norm
    x = tanh(alpha * h) * weight + bias of every row (of `rows` only, if given: h then stays as it is), in one pass."""
    _cuda(h, "h", torch.float32)
    n_total, hidden = h.shape
    y = z = zb = None
    z_stride = 0
    if isinstance(delta, GatedDelta):
        y, z, zb = delta.y, delta.z, delta.bias
        _cuda(z, "gate", contiguous=False); _cuda(zb, "gate bias")
        if z.shape != h.shape or z.stride(1) != 1 or zb.numel() != hidden:
            raise KernelError("gated residual: the gate has the stream's shape, its bias one row")
        z_stride = z.stride(0)
    elif delta is not None:
        y = delta if isinstance(delta, torch.Tensor) else delta.tensor()
    if y is not None:
        _cuda(y, "delta")
        if y.shape != h.shape:
            raise KernelError("delta and h differ in shape")
    out = None
    if weight is not None:
        _cuda(weight, "weight"); _cuda(bias, "bias", weight.dtype)
        if weight.numel() != hidden or bias.numel() != hidden:
            raise KernelError("dynamic-tanh norm: weight and bias have one row's size")
        if zb is not None and zb.dtype != weight.dtype:
            zb = zb.to(weight.dtype)
        n_out = n_total if rows is None else rows.numel()
        out = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    elif rows is not None:
        raise KernelError("gated_add_dyt: rows are for the norm")
    else:
        n_out = n_total
        if y is None:
            return None
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
    w_code = _code(weight, "weight") if weight is not None else (_code(zb, "gate bias") if zb is not None else 0)
    f = _fn("dyt", "jv_gated_add_dyt", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p, c_float,
                                        c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(h.data_ptr(), _ptr(rows), _ptr(y), 0 if y is None else _code(y, "delta"), _ptr(z),
             0 if z is None else _code(z, "gate"), z_stride, _ptr(zb), float(alpha), _ptr(weight), _ptr(bias), w_code,
             _ptr(out), 0 if out is None else _code(out, "out"), n_out, n_total, hidden, _status_ptr(h.device), _stream()),
           "gated_add_dyt")
    return out


def add_row(h: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """h[n, :] += vec for every row of the float32 stream."""
    _cuda(h, "h", torch.float32); _cuda(vec, "vec")
    if vec.numel() != h.shape[1]:
        raise KernelError("add_row: the vector has one row's size")
    f = _fn("dyt", "jv_add_row", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(h.data_ptr(), vec.data_ptr(), _code(vec, "vec"), h.shape[0], h.shape[1], _stream()), "add_row")
    return h


def norm_mean2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float,
               coef: float = 0.5) -> torch.Tensor:
    """coef * (unit(a) * wa + unit(b) * wb) as float32, unit(y) = y / sqrt(mean(y^2) + eps) over a row."""
    _cuda(a, "a"); _cuda(b, "b", a.dtype); _cuda(wa, "wa"); _cuda(wb, "wb", wa.dtype)
    n, hidden = a.shape
    if b.shape != a.shape or wa.numel() != hidden or wb.numel() != hidden:
        raise KernelError("norm_mean2: shapes do not fit")
    out = torch.empty((n, hidden), dtype=torch.float32, device=a.device)
    f = _fn("dyt", "jv_norm_mean2", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
                                     c_float, c_void_p])
    _check(f(a.data_ptr(), b.data_ptr(), _code(a, "a"), wa.data_ptr(), wb.data_ptr(), _code(wa, "wa"), out.data_ptr(), n,
             hidden, float(eps), float(coef), _stream()), "norm_mean2")
    return out


# ------------------------------------------------ matrix states carried from token to token (csrc/recurrent.cu)
SCAN_MAX_KEY = 256


def delta_prepare(proj: torch.Tensor, r_off: int, k_off: int, a_off: int, zw: torch.Tensor, a_bias: torch.Tensor,
                  w_bias: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    """Per token and head the vectors (r, k, w, u, b) of the generalized delta rule as float32 [n, heads, 5, dim]:
    w = exp(-e^(-1/2) sigmoid(zw + w_bias)), u = k / sqrt(|k|^2 + 1e-6), b = sigmoid(z_a + a_bias) * u."""
    _cuda(proj, "proj", contiguous=False); _cuda(zw, "zw", proj.dtype, contiguous=False)
    _cuda(a_bias, "a_bias"); _cuda(w_bias, "w_bias", a_bias.dtype)
    n = proj.shape[0]
    if proj.stride(1) != 1 or zw.stride(1) != 1 or zw.shape != (n, heads * dim) or \
            max(r_off, k_off, a_off) + heads * dim > proj.shape[1] or a_bias.numel() != heads * dim or \
            w_bias.numel() != heads * dim:
        raise KernelError("delta_prepare: shapes do not fit")
    packed = torch.empty((n, heads, 5, dim), dtype=torch.float32, device=proj.device)
    f = _fn("recurrent", "jv_delta_prepare", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong,
                                              c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(proj.data_ptr(), _code(proj, "proj"), proj.stride(0), r_off, k_off, a_off, zw.data_ptr(), zw.stride(0),
             a_bias.data_ptr(), w_bias.data_ptr(), _code(a_bias, "a_bias"), packed.data_ptr(), n, heads, dim, _stream()),
           "delta_prepare")
    return packed


def memory_gates(proj: torch.Tensor, q_off: int, k_off: int, i_off: int, f_off: int, i_bias: torch.Tensor,
                 f_bias: torch.Tensor, cap: float, q_scale: float, state_m: torch.Tensor, cu_seqlens: torch.Tensor,
                 slots: torch.Tensor, n_entries: int, heads: int, dim: int):
    """The gates of a matrix memory with exponential gating: the running maximum `state_m` [slots, heads] (a view of
    the state rows) is scanned over every entry's tokens, then all tokens at once are prepared.  Returns (packed
    float32 [n, heads, 3, dim]: the scaled query, the key times its input gate, the decay; gates float32 [n, heads,
    4]: decay, input gate, running maximum, and a place that `state_scan` fills with n . q)."""
    _cuda(proj, "proj", contiguous=False); _cuda(i_bias, "i_bias"); _cuda(f_bias, "f_bias", i_bias.dtype)
    _cuda(state_m, "state_m", torch.float32, contiguous=False)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(slots, "slots", torch.int32)
    n = proj.shape[0]
    if proj.stride(1) != 1 or state_m.stride(1) != 1 or state_m.shape[1] != heads or dim > SCAN_MAX_KEY or \
            max(q_off, k_off) + heads * dim > proj.shape[1] or max(i_off, f_off) + heads > proj.shape[1]:
        raise KernelError("memory_gates: shapes do not fit")
    packed = torch.empty((n, heads, 3, dim), dtype=torch.float32, device=proj.device)
    gates = torch.empty((n, heads, 4), dtype=torch.float32, device=proj.device)
    f = _fn("recurrent", "jv_memory_gates", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                             c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(proj.data_ptr(), _code(proj, "proj"), proj.stride(0), q_off, k_off, i_off, f_off, i_bias.data_ptr(),
             f_bias.data_ptr(), _code(i_bias, "i_bias"), float(cap), float(q_scale), gates.data_ptr(), packed.data_ptr(),
             state_m.data_ptr(), state_m.stride(0), cu_seqlens.data_ptr(), slots.data_ptr(), state_m.shape[0], n_entries,
             n, heads, dim, _status_ptr(proj.device), _stream()), "memory_gates", launches=2)
    return packed, gates


SCAN_SEGMENT = 64          # tokens of a segment when long entries are scanned in segments side by side
SCAN_SEGMENT_MEAN = 32     # ... which happens when the entries of a step have this many tokens on average, at least


def state_scan(packed: torch.Tensor, v: torch.Tensor, v_off: int, state: torch.Tensor, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, n_entries: int, value_dim: int, state_n: torch.Tensor | None = None,
               gates: torch.Tensor | None = None, segment: int | None = None) -> torch.Tensor:
    """S <- diag(w) S - b (u^T S) + k v^T and o = S^T r, token after token of every entry, for the per-head states
    `state` [slots, >= heads * dim * value_dim] float32 (a view of the state rows); `packed` [n, heads, 5 or 3, dim]
    holds (r, k, w, u, b) or, without the removal term, (r, k, w); the values are columns `v_off`.. of the rows of
    `v`.  Returns o [n, heads * value_dim] float32.  With `state_n` [slots, heads * dim] (a view of the same rows) the
    state has one more column whose value is 1 at every token (a normaliser n <- w n + k); its output n . r goes to
    the fourth place of `gates` [n, heads, 4].

    A step whose entries are long runs them in segments of `segment` tokens side by side (None: `SCAN_SEGMENT` when
    the step has 4 segments' tokens and `SCAN_SEGMENT_MEAN` tokens an entry; 0: never): every segment first runs from
    a zero state and records what it does to a state that comes in, the segments of an entry are chained, and every
    segment runs again from its true start for the outputs.  The result differs from the token-by-token order by
    32-bit rounding only."""
    _cuda(packed, "packed", torch.float32); _cuda(v, "v", contiguous=False)
    _cuda(state, "state", torch.float32, contiguous=False)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(slots, "slots", torch.int32)
    n, heads, nv, dim = packed.shape
    if nv not in (3, 5) or v.shape[0] != n or v.stride(1) != 1 or v_off + heads * value_dim > v.shape[1] or \
            state.stride(1) != 1 or state.shape[1] < heads * dim * value_dim or dim > SCAN_MAX_KEY:
        raise KernelError("state_scan: shapes do not fit")
    nq = None
    if state_n is not None:
        _cuda(state_n, "state_n", torch.float32, contiguous=False); _cuda(gates, "gates", torch.float32)
        if nv != 3 or state_n.stride(0) != state.stride(0) or state_n.stride(1) != 1 or state_n.shape[1] != heads * dim or \
                state_n.shape[0] != state.shape[0] or tuple(gates.shape) != (n, heads, 4):
            raise KernelError("state_scan: the normaliser does not fit")
        nq = gates.data_ptr() + 3 * 4
    out = torch.empty((n, heads * value_dim), dtype=torch.float32, device=packed.device)
    if segment is None:
        # with the removal term a segment carries `dim` more columns and the chain is a matrix product a segment: at
        # the sizes measured (32 heads of 64, 2,048 tokens) the three launches take longer than the one
        segment = SCAN_SEGMENT if nv == 3 and n >= 4 * SCAN_SEGMENT and n >= SCAN_SEGMENT_MEAN * n_entries else 0
    if nv == 5 and 4 * dim * (64 + (dim + 3) // 4 * 4 + 4) > 200 * 1024:
        segment = 0          # the kernel that chains segments keeps a [dim][dim] transition in shared memory
    max_segments, seg_local, seg_start = 0, None, None
    if segment > 0:
        max_segments = n // segment + n_entries
        v_tot = value_dim + (1 if state_n is not None else 0) + (dim if nv == 5 else 1)
        seg_local = torch.empty((2, max_segments, heads, dim, v_tot), dtype=torch.float32, device=packed.device)
        seg_start = seg_local[1]
    f = _fn("recurrent", "jv_state_scan", [c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p,
                                           c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                           c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(packed.data_ptr(), 1 if nv == 5 else 0, v.data_ptr(), _code(v, "v"), v.stride(0), v_off, out.data_ptr(),
             state.data_ptr(), state.stride(0), cu_seqlens.data_ptr(), slots.data_ptr(), state.shape[0], n_entries, heads,
             dim, value_dim, _ptr(state_n), nq, 4, int(segment), max_segments, _ptr(seg_local), _ptr(seg_start),
             _status_ptr(packed.device), _stream()), "state_scan", launches=3 if segment > 0 else 1)
    return out


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, heads: int,
                   value_dim: int, eps: float, gates: torch.Tensor | None = None) -> torch.Tensor:
    """Each head of `o` [n, heads * value_dim] float32 divided by its root mean square, times `weight` [heads *
    value_dim], times sigmoid(gate) (rows of `out`'s type, possibly a column range), written to `out` (possibly a
    column range).  With `gates` [n, heads, 4] = (-, -, m, n . q) each head is first divided by
    max(|n . q|, exp(-m)) + 1e-6."""
    _cuda(o, "o", torch.float32); _cuda(weight, "weight"); _cuda(out, "out", contiguous=False)
    n = o.shape[0]
    if o.shape[1] != heads * value_dim or out.shape != o.shape or out.stride(1) != 1 or weight.numel() != o.shape[1]:
        raise KernelError("head_norm_gate: shapes do not fit")
    g_stride = 0
    if gate is not None:
        _cuda(gate, "gate", out.dtype, contiguous=False)
        if gate.shape != o.shape or gate.stride(1) != 1:
            raise KernelError("head_norm_gate: the gate has the heads' shape")
        g_stride = gate.stride(0)
    if gates is not None:
        _cuda(gates, "gates", torch.float32)
        if tuple(gates.shape) != (n, heads, 4):
            raise KernelError("head_norm_gate: gates are [n, heads, 4]")
    f = _fn("recurrent", "jv_head_norm_gate", [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_longlong,
                                               c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(o.data_ptr(), weight.data_ptr(), _code(weight, "weight"), _ptr(gate), g_stride, out.data_ptr(),
             _code(out, "out"), out.stride(0), n, heads, value_dim, float(eps), _ptr(gates), _stream()), "head_norm_gate")
    return out


# ------------------------------------------------ short convolutions with state (csrc/short_conv.cu)
SHORT_CONV_MAX_TAPS = 8
SHORT_CONV_ACTS = {None: 0, "silu": 1}


def short_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, n_entries: int, out_dtype: torch.dtype, bias: torch.Tensor | None = None,
               act: str | None = None, residual: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """A causal convolution over time on each channel of `x` [n, channels] (rows possibly a column range of a wider
    tensor), `weight` [channels, taps] with the last column on the current token; out = act(conv + bias), or with
    `residual` x + conv.  `state` [slots, (taps - 1) * channels] float32 (a view of the state rows) holds the last
    taps - 1 inputs of every sequence and is renewed; a zero row is a sequence's start.  32-bit arithmetic."""
    _cuda(x, "x", contiguous=False); _cuda(weight, "weight")
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(slots, "slots", torch.int32)
    n, channels = x.shape
    taps = weight.shape[1]
    if x.stride(1) != 1 or weight.shape[0] != channels or not 1 <= taps <= SHORT_CONV_MAX_TAPS or act not in SHORT_CONV_ACTS:
        raise KernelError("short_conv: shapes do not fit")
    if bias is not None:
        _cuda(bias, "bias", weight.dtype)
        if bias.numel() != channels or residual:
            raise KernelError("short_conv: a bias per channel, and none where the convolution is added to its input")
    n_slots = stride = 0
    if taps > 1:
        _cuda(state, "state", torch.float32, contiguous=False)
        if state.stride(1) != 1 or state.shape[1] != (taps - 1) * channels:
            raise KernelError("short_conv: the state holds taps - 1 inputs of every channel")
        n_slots, stride = state.shape[0], state.stride(0)
    if out is None:
        out = torch.empty((n, channels), dtype=out_dtype, device=x.device)
    _cuda(out, "out", out_dtype, contiguous=False)
    if out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("short_conv: out has the shape of x")
    f = _fn("short_conv", "jv_short_conv", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p,
                                            c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), _code(x, "x"), x.stride(0), out.data_ptr(), _code(out, "out"), out.stride(0),
             weight.data_ptr(), _ptr(bias), _code(weight, "weight"), _ptr(state) if taps > 1 else 0, stride,
             cu_seqlens.data_ptr(), slots.data_ptr(), n_entries, n_slots, n, channels, taps, SHORT_CONV_ACTS[act],
             1 if residual else 0, _status_ptr(x.device), _stream()), "short_conv")
    return out


# ------------------------------------------------ heads prepared one by one (csrc/head_prepare.cu)
def head_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, positions: torch.Tensor,
                 token_entry: torch.Tensor, block_table: torch.Tensor, freq: torch.Tensor | None, interleaved: bool,
                 q_norm_w, k_norm_w, eps: float, value_norm: bool, value_freq: torch.Tensor | None, k_cache, v_cache,
                 n_q_heads: int, n_k_heads: int, n_v_heads: int, key_dim: int, value_dim: int) -> None:
    """Per head: RMSNorm of queries and keys with one weight vector [key_dim] shared by the heads (or none), rotation of
    the first 2 * len(freq) elements (pairs in halves or `interleaved`); values divided by their root mean square
    (`value_norm`) and rotated by their own position over 2 * len(value_freq) elements; keys and values written to
    their pages (both caches None: queries only).  32-bit arithmetic."""
    _cuda(proj, "proj", contiguous=False); _cuda(q_out, "q_out", proj.dtype)
    _cuda(positions, "positions", torch.int32); _cuda(token_entry, "token_entry", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    n = proj.shape[0]
    if proj.stride(1) != 1 or q_out.shape != (n, n_q_heads * key_dim):
        raise KernelError("head_prepare: shapes do not fit")
    rot = v_rot = 0
    if freq is not None:
        _cuda(freq, "freq", torch.float32)
        rot = 2 * freq.numel()
    if value_freq is not None:
        _cuda(value_freq, "value_freq", torch.float32)
        v_rot = 2 * value_freq.numel()
    w_code = 0
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            _cuda(w, "norm weight")
            if w.numel() != key_dim:
                raise KernelError("head_prepare: the norm's weight has the head's size")
            w_code = _code(w, "norm weight")
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("head_prepare: both norm weights have one type")
    writes = k_cache is not None
    page_size = num_pages = 1
    if writes:
        _cuda(k_cache, "k_cache", proj.dtype); _cuda(v_cache, "v_cache", proj.dtype)
        if k_cache.shape[2:] != (n_k_heads, key_dim) or v_cache.shape[2:] != (n_v_heads, value_dim) or \
                k_cache.shape[:2] != v_cache.shape[:2]:
            raise KernelError("head_prepare: the caches do not fit the heads")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
        if max(k_off + n_k_heads * key_dim, v_off + n_v_heads * value_dim) > proj.shape[1]:
            raise KernelError("head_prepare: the projection row is too short")
    if q_off + n_q_heads * key_dim > proj.shape[1]:
        raise KernelError("head_prepare: the projection row is too short")
    f = _fn("head_prepare", "jv_head_prepare",
            [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(proj.data_ptr(), _code(proj, "proj"), proj.stride(0), q_off, k_off, v_off, q_out.data_ptr(),
             positions.data_ptr(), token_entry.data_ptr(), block_table.data_ptr(), block_table.shape[1], _ptr(freq), rot,
             _ptr(value_freq), v_rot, 1 if interleaved else 0, _ptr(q_norm_w), _ptr(k_norm_w), w_code, float(eps),
             1 if value_norm else 0, _ptr(k_cache) if writes else 0, _ptr(v_cache) if writes else 0, n, n_q_heads,
             n_k_heads, n_v_heads, key_dim, value_dim, page_size, num_pages, _status_ptr(proj.device), _stream()),
           "head_prepare")


def head_rotate(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, interleaved: bool, heads: int, dim: int,
                sign: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Every head of `x` [n, heads * dim] turned by sign * position * freq[j] over its first 2 * len(freq) elements, in
    place or into `out` (rows possibly a column range; any of the two types)."""
    _cuda(x, "x", contiguous=False); _cuda(positions, "positions", torch.int32); _cuda(freq, "freq", torch.float32)
    out = x if out is None else _cuda(out, "out", contiguous=False)
    if x.shape[1] != heads * dim or out.shape != x.shape or x.stride(1) != 1 or out.stride(1) != 1 or 2 * freq.numel() > dim:
        raise KernelError("head_rotate: shapes do not fit")
    f = _fn("head_prepare", "jv_head_rotate", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p,
                                               c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
    _check(f(x.data_ptr(), _code(x, "x"), x.stride(0), out.data_ptr(), _code(out, "out"), out.stride(0),
             positions.data_ptr(), freq.data_ptr(), 2 * freq.numel(), 1 if interleaved else 0, float(sign), x.shape[0],
             heads, dim, _stream()), "head_rotate")
    return out


def rms_rows(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """Rows of `x` [n, width] (possibly a column range of a wider tensor) divided by their root mean square, times
    `weight`; 32-bit arithmetic, the result in x's type."""
    _cuda(x, "x", contiguous=False)
    if x.stride(1) != 1:
        raise KernelError("rms_rows: rows have unit column stride")
    if weight is not None:
        _cuda(weight, "weight")
        if weight.numel() != x.shape[1]:
            raise KernelError("rms_rows: the weight has the rows' width")
    out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    f = _fn("head_prepare", "jv_rms_rows", [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_int, c_float,
                                            c_int, c_int, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), _code(x, "x"), _ptr(weight),
             0 if weight is None else _code(weight, "weight"), float(eps), x.shape[0], x.shape[1], _stream()), "rms_rows")
    return out


# ------------------------------------------------ state-space mixer: around the state scan (csrc/mamba2.cu)
def mamba_prepare(xbc: torch.Tensor, b_off: int, c_off: int, dt_raw: torch.Tensor, dt_bias: torch.Tensor,
                  a_log: torch.Tensor, heads: int, groups: int, state: int) -> torch.Tensor:
    """Per token and head (C_g, softplus(dt + dt_bias) * B_g, exp(-exp(A_log) * dt)) as float32 [n, heads, 3, state]:
    query, key and decay of `state_scan`.  B and C are [groups, state] column ranges of the rows `xbc`."""
    _cuda(xbc, "xbc", contiguous=False); _cuda(dt_raw, "dt", xbc.dtype, contiguous=False)
    _cuda(dt_bias, "dt_bias"); _cuda(a_log, "A_log", dt_bias.dtype)
    n = xbc.shape[0]
    if xbc.stride(1) != 1 or dt_raw.stride(1) != 1 or dt_raw.shape != (n, heads) or heads % groups or \
            max(b_off, c_off) + groups * state > xbc.shape[1] or dt_bias.numel() != heads or a_log.numel() != heads:
        raise KernelError("mamba_prepare: shapes do not fit")
    packed = torch.empty((n, heads, 3, state), dtype=torch.float32, device=xbc.device)
    f = _fn("mamba2", "jv_mamba_prepare", [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_longlong, c_void_p,
                                           c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(xbc.data_ptr(), _code(xbc, "xbc"), xbc.stride(0), b_off, c_off, dt_raw.data_ptr(), dt_raw.stride(0),
             dt_bias.data_ptr(), a_log.data_ptr(), _code(dt_bias, "dt_bias"), packed.data_ptr(), n, heads, groups, state,
             _stream()), "mamba_prepare")
    return packed


def mamba_finish(o: torch.Tensor, x: torch.Tensor, z: torch.Tensor, skip: torch.Tensor, weight: torch.Tensor,
                 out: torch.Tensor, heads: int, value_dim: int, norm_groups: int, eps: float) -> torch.Tensor:
    """y = (o + skip_h * x) * silu(z), divided by the root mean square of each of its `norm_groups` equal parts, times
    `weight`; o float32 [n, heads * value_dim], x and z column ranges of rows in the compute type; written to `out`."""
    _cuda(o, "o", torch.float32); _cuda(x, "x", contiguous=False); _cuda(z, "z", x.dtype, contiguous=False)
    _cuda(skip, "skip"); _cuda(weight, "weight", skip.dtype); _cuda(out, "out", x.dtype, contiguous=False)
    n, inner = o.shape
    if inner != heads * value_dim or inner % norm_groups or x.shape != o.shape or z.shape != o.shape or \
            out.shape != o.shape or x.stride(1) != 1 or z.stride(1) != 1 or out.stride(1) != 1 or skip.numel() != heads or \
            weight.numel() != inner:
        raise KernelError("mamba_finish: shapes do not fit")
    f = _fn("mamba2", "jv_mamba_finish", [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                          c_int, c_void_p, c_longlong, c_float, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(o.data_ptr(), x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0), _code(x, "x"), skip.data_ptr(),
             weight.data_ptr(), _code(skip, "skip"), out.data_ptr(), out.stride(0), float(eps), n, heads, value_dim,
             norm_groups, _stream()), "mamba_finish")
    return out


# ------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor) -> torch.Tensor:
    """One token per row of float32 logits: argmax where temperature is 0, else a draw from
    softmax(logits / temperature) that depends on (seed, counter) of the row only."""
    _cuda(logits, "logits", torch.float32); _cuda(temperature, "temperature", torch.float32)
    _cuda(seeds, "seeds", torch.int64); _cuda(counters, "counters", torch.int64)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    chunks = min(128, max(1, -(-vocab // 2048)))
    part_v = torch.empty(rows * chunks, dtype=torch.float32, device=logits.device)
    part_i = torch.empty(rows * chunks, dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "jv_sample", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p])
    _check(f(logits.data_ptr(), rows, vocab, temperature.data_ptr(), seeds.data_ptr(), counters.data_ptr(),
             part_v.data_ptr(), part_i.data_ptr(), out.data_ptr(), _stream()), "sample", launches=2)
    return out
