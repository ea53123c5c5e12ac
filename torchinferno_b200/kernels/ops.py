"""Python faces of the CUDA kernels.

Each function checks device, dtype, contiguity and shapes, then calls the C
entry point on torch's current stream.  A refusal by a kernel (a size it does
not take) raises :class:`KernelError`; nothing falls back to another path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from torchinferno_b200.kernels.library import load_library

F32, BF16 = 0, 1

_ERRORS = {
    -1: "unknown dtype code",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride that is not aligned as required",
    -4: "needs more shared memory than an SM offers",
    -5: "null pointer or inconsistent arguments",
    -6: "the device-side wait limit was reached (kernel gave up)",
    -7: "needs more scratch than the library's built-in array holds",
}


class KernelError(RuntimeError):
    pass


_counter = {"launches": 0}


def set_dependent_launch(on: bool) -> bool:
    """Programmatic dependent launch of the library's small kernels (on by default): a kernel may be placed on
    the SMs while the one before it drains and waits there for its data.  Returns the setting before.  A
    captured graph keeps what was set when it was captured."""
    return bool(lib().tib_set_dependent_launch(c_int(1 if on else 0)))


KERNEL_CLASSES = ("norm", "qkv", "rope_append", "attention_prefill", "attention_decode", "o", "gate_up", "swiglu", "down")


def set_kernel_timers(on: bool) -> bool:
    """CUDA-event timers around every launch of a natively issued block, by kernel class (off by default; a step
    captured in a graph records nothing).  Returns the setting before."""
    return bool(lib().tib_kernel_timers(c_int(1 if on else 0)))


def read_kernel_timers(reset: bool = False) -> dict[str, dict[str, float]]:
    """{class: {"ms": total, "launches": n}} of what the timers have recorded; waits for the recorded events."""
    n = len(KERNEL_CLASSES)
    ms, counts = (ctypes.c_double * n)(), (ctypes.c_longlong * n)()
    lib().tib_kernel_timers_read(ms, counts, c_int(n), c_int(1 if reset else 0))
    return {name: {"ms": float(ms[i]), "launches": int(counts[i])} for i, name in enumerate(KERNEL_CLASSES)}


def count_launches(n: int) -> None:
    """Launches made by a native call that issues several kernels."""
    _counter["launches"] += n


def launch_count() -> int:
    """How many kernels of this library were launched by this process so far."""
    return _counter["launches"]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 or bfloat16)")


def _check(name: str, status: int) -> None:
    _counter["launches"] += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{name}: refused: {_ERRORS.get(status, status)}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _stream() -> c_void_p:
    # (the raw handle of the current stream of the current device: a fraction of the cost of
    # torch.cuda.current_stream(), which is asked for at every launch)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_signatures_set = False


def lib() -> ctypes.CDLL:
    global _signatures_set
    library = load_library()
    if not _signatures_set:
        for fn in ("tib_embedding", "tib_add_rmsnorm", "tib_rmsnorm", "tib_swiglu", "tib_cast",
                   "tib_scatter_i32", "tib_decode_inputs", "tib_sample_records", "tib_rope_append", "tib_paged_attention_simt", "tib_gemm_f32", "tib_sample",
                   "tib_attention_mma_supports", "tib_prefill_attention", "tib_decode_attention",
                   "tib_prefill_attention_tcgen05", "tib_prefill_attention_tcgen05_supports",
                   "tib_decode_attention_tma", "tib_decode_attention_tma_rope", "tib_decode_attention_tma_supports", "tib_set_dependent_launch",
                   "tib_kernel_timers", "tib_kernel_timers_read",
                   "tib_blas_init", "tib_blas_gemm", "tib_gemm_tcgen05_2cta", "tib_gemm_tcgen05_2cta_supports",
                   "tib_gemm_tcgen05", "tib_gemm_tcgen05_supports",
                   "tib_gemm_tcgen05_swapab", "tib_gemm_tcgen05_swapab_supports", "tib_gemm_decode", "tib_gemm_decode_supports",
                   "tib_plan_attention", "tib_plan_product", "tib_blas_gemm_batched",
                   "tib_add_pair", "tib_unit_norm_add", "tib_sigmoid_gate", "tib_gelu_gate_table", "tib_relu_squared",
                   "tib_scale_f32", "tib_pair_rows", "tib_add_vector", "tib_linear_attention", "tib_linear_attention_chunk",
                   "tib_latent_append", "tib_latent_attention", "tib_latent_attention_splits", "tib_moe_route", "tib_moe_group", "tib_router_logits",
                   "tib_moe_expert_product", "tib_moe_combine", "tib_glu_clamp", "tib_layernorm", "tib_layernorm_tail",
                   "tib_qk_norm_append", "tib_sigmoid_attention", "tib_sigmoid_attention_takes_mma", "tib_gated_recurrence",
                   "tib_softcap_f32", "tib_short_conv", "tib_ssd_scan", "tib_ssd_scan_max_state", "tib_ssd_scan_run", "tib_gated_group_norm",
                   "tib_rotary_kv_append", "tib_pool_blocks", "tib_pooled_window_attention", "tib_hyper_step",
                   "tib_pooled_window_attention_splits", "tib_pooled_window_attention_part_floats"):
            getattr(library, fn).restype = c_int
        _signatures_set = True
    return library


# ---------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = float(table[ids[t]]): the residual stream starts in 32-bit."""
    _need(ids, "ids", torch.int32), _need(table, "table"), _need(out, "out", torch.float32)
    n, (vocab, hidden) = ids.numel(), table.shape
    if out.shape != (n, hidden):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, wanted {(n, hidden)}")
    _check("embedding", lib().tib_embedding(_ptr(ids), _ptr(table), _ptr(out), c_int(n), c_int(hidden),
                                            c_int(vocab), c_int(_code(table.dtype)), _stream()))
    return out


def add_rmsnorm(delta: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (fp32, in place, when rows is None); out = rmsnorm(residual) * weight.

    With ``rows`` only those source rows are read, the residual is left as it
    is and ``out`` has one row per index.
    """
    _need(residual, "residual", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    hidden = residual.shape[-1]
    if delta is not None:
        _need(delta, "delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("add_rmsnorm: delta and residual differ in shape")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = residual.shape[0] if rows is None else rows.numel()
    if out.shape != (n_out, hidden) or weight.numel() != hidden:
        raise KernelError(f"add_rmsnorm: out {tuple(out.shape)} / weight {tuple(weight.shape)} do not fit {(n_out, hidden)}")
    _check("add_rmsnorm", lib().tib_add_rmsnorm(_ptr(delta), _ptr(residual), _ptr(rows), _ptr(weight), _ptr(out),
                                                c_int(n_out), c_int(hidden), c_float(eps),
                                                c_int(_code(out.dtype)), _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """RMSNorm over the last dimension of rows held in the activation type (``x`` may be a column slice of wider
    2-D rows; ``out`` is contiguous)."""
    _need(weight, "weight", torch.float32), _need(out, "out", x.dtype)
    hidden = x.shape[-1]
    if x.dim() == 2 and not x.is_contiguous():
        _rows_of(x, "x")
        ldx = x.stride(0)
    else:
        _need(x, "x")
        ldx = hidden
    n_rows = x.numel() // hidden if hidden else 0
    if out.shape != x.shape or weight.numel() != hidden:
        raise KernelError("rmsnorm: shapes do not fit")
    _check("rmsnorm", lib().tib_rmsnorm(_ptr(x), c_int64(ldx), _ptr(weight), _ptr(out), c_int(n_rows), c_int(hidden),
                                        c_float(eps), c_int(_code(x.dtype)), _stream()))
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out = silu(gate) * up, silu and product in fp32; a row of ``gate_up`` holds the I gates, then the I ups,
    or (``interleaved``) gate i and up i side by side."""
    _need(gate_up, "gate_up"), _need(out, "out", gate_up.dtype)
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2):
        raise KernelError("swiglu: shapes do not fit")
    _check("swiglu", lib().tib_swiglu(_ptr(gate_up), _ptr(out), c_int(n), c_int(two_i // 2),
                                      c_int(_code(gate_up.dtype)), c_int(int(interleaved)), _stream()))
    return out


def cast(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(x, "x"), _need(out, "out")
    if x.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check("cast", lib().tib_cast(_ptr(x), _ptr(out), c_int64(x.numel()), c_int(_code(x.dtype)),
                                  c_int(_code(out.dtype)), _stream()))
    return out


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, pool: torch.Tensor | None, positions: torch.Tensor,
                token_slot: torch.Tensor | None, block_table: torch.Tensor | None, inv_freq: torch.Tensor,
                heads: int, kv_heads: int, head_dim: int, *, rot_dim: int | None = None,
                interleaved: bool = False, write_kv: bool = True,
                error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate q into ``q_out``; rotate k and copy v into the layer's pages.

    ``qkv``: [tokens, (heads + 2 kv_heads) * head_dim]; ``pool``: the layer's pages
    [pages, 2, kv_heads, page_size, head_dim]; ``block_table``: [slots, max_pages] int32.
    """
    _need(qkv, "qkv"), _need(q_out, "q_out", qkv.dtype), _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    n = qkv.shape[0]
    rot = head_dim if rot_dim is None else rot_dim
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim or q_out.numel() != n * heads * head_dim:
        raise KernelError("rope_append: qkv / q_out widths do not fit the head counts")
    if inv_freq.numel() != rot // 2 or positions.numel() != n:
        raise KernelError("rope_append: inv_freq or positions have the wrong length")
    page_size = page_stride = num_pages = table_stride = 0
    if write_kv:
        if pool is None or token_slot is None or block_table is None:
            raise KernelError("rope_append: pool, token_slot and block_table are needed to write the cache")
        _need(pool, "pool", qkv.dtype), _need(token_slot, "token_slot", torch.int32)
        _need(block_table, "block_table", torch.int32)
        if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
            raise KernelError(f"rope_append: pool shape {tuple(pool.shape)} does not fit")
        num_pages, page_size = pool.shape[0], pool.shape[3]
        page_stride = pool.stride(0)
        table_stride = block_table.stride(0)
    _check("rope_append", lib().tib_rope_append(
        _ptr(qkv), _ptr(q_out), _ptr(pool), _ptr(positions), _ptr(token_slot), _ptr(block_table),
        c_int(table_stride), _ptr(inv_freq), c_int(n), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(rot), c_int(int(interleaved)), c_int(page_size), c_int64(page_stride), c_int(num_pages),
        c_int(int(write_kv)), _ptr(error_word), c_int(_code(qkv.dtype)), _stream()))
    return q_out


def paged_attention_simt(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                         kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor,
                         n_entries: int, max_q_len: int, heads: int, kv_heads: int, head_dim: int,
                         scale: float, window: int = 0, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of a ragged batch over the paged cache, on CUDA cores."""
    _need(q, "q"), _need(pool, "pool", q.dtype), _need(out, "out", q.dtype)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"paged_attention: pool shape {tuple(pool.shape)} does not fit")
    if q.numel() != out.numel() or q.numel() % (heads * head_dim):
        raise KernelError("paged_attention: q / out do not fit the head counts")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("paged_attention: entry arrays are shorter than n_entries")
    _check("paged_attention_simt", lib().tib_paged_attention_simt(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads),
        c_int(head_dim), c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window),
        c_float(scale), _ptr(error_word), c_int(_code(q.dtype)), _stream()))
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (fp32) = x[M, K] . w[N, K]^T with fp32 FMAs in fixed k order (rows of all three at any stride)."""
    if out.dtype != torch.float32:
        raise KernelError(f"out must be float32, got {out.dtype}")
    for name, t in (("x", x), ("w", w), ("out", out)):
        if not t.is_cuda or t.stride(-1) != 1 or t.dim() != 2:
            raise KernelError(f"gemm_f32: {name} must be a 2-D CUDA tensor with unit inner stride")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_f32", lib().tib_gemm_f32(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                          c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                          c_int(_code(x.dtype)), c_int(_code(w.dtype)), _stream()))
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           seeds: torch.Tensor | None = None, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Token ids from fp32 logits: greedy where temperature <= 0, else seeded Gumbel-max."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a 2-D fp32 CUDA tensor with unit inner stride")
    _need(out, "out", torch.int32)
    n, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
    if seeds is not None:
        _need(seeds, "seeds", torch.int64)
    if positions is not None:
        _need(positions, "positions", torch.int32)
    for t in (temperature, seeds, positions):
        if t is not None and t.numel() < n:
            raise KernelError("sample: a per-row array is shorter than the number of rows")
    if out.numel() < n:
        raise KernelError("sample: out is too short")
    _check("sample", lib().tib_sample(_ptr(logits), c_int64(logits.stride(0)), _ptr(temperature), _ptr(seeds),
                                      _ptr(positions), _ptr(out), c_int(n), c_int(vocab), _stream()))
    return out


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """dst.view(-1)[index[i]] = value[i]; applies queued block-table changes."""
    _need(dst, "dst", torch.int32), _need(index, "index", torch.int32), _need(value, "value", torch.int32)
    if index.numel() != value.numel():
        raise KernelError("scatter_i32: index and value differ in length")
    _check("scatter_i32", lib().tib_scatter_i32(_ptr(dst), _ptr(index), _ptr(value), c_int(index.numel()),
                                                c_int64(dst.numel()), _stream()))
    return dst


RECORD_WORDS = 8          # int32 words of a request's record (csrc/common.cuh: TibRequestRecord)
REC_LENGTH, REC_LAST_TOKEN, REC_SEED_LO, REC_SEED_HI, REC_TEMPERATURE, REC_DRAWN = range(6)


def _need_records(records: torch.Tensor) -> None:
    _need(records, "records", torch.int32)
    if records.dim() != 2 or records.shape[1] != RECORD_WORDS:
        raise KernelError(f"records must be [slots, {RECORD_WORDS}] int32")


def sample_records(logits: torch.Tensor, out: torch.Tensor, records: torch.Tensor, record_slots: torch.Tensor,
                   history: torch.Tensor | None = None) -> torch.Tensor:
    """As :func:`sample`, every row's temperature, seed and position taken from the record of its request
    (``record_slots[row]``); the drawn token also goes into that record as the request's next input token."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a 2-D fp32 CUDA tensor with unit inner stride")
    _need(out, "out", torch.int32), _need_records(records), _need(record_slots, "record_slots", torch.int32)
    n, vocab = logits.shape
    if history is not None:
        _need(history, "history", torch.int32)
    if out.numel() < n or record_slots.numel() < n or (history is not None and history.numel() < n):
        raise KernelError("sample: a per-row array is shorter than the number of rows")
    _check("sample", lib().tib_sample_records(_ptr(logits), c_int64(logits.stride(0)), _ptr(records), _ptr(record_slots),
                                              c_int(records.shape[0]), _ptr(out), _ptr(history), c_int(n), c_int(vocab), _stream()))
    return out


def decode_inputs(records: torch.Tensor, slots: torch.Tensor, token_ids: torch.Tensor, positions: torch.Tensor) -> None:
    """token_ids[i], positions[i] = next token and position of the request in slot slots[i]; its record moves on by one."""
    n = slots.numel()
    _need_records(records)
    for name, t in (("slots", slots), ("token_ids", token_ids), ("positions", positions)):
        _need(t, name, torch.int32)
        if t.numel() < n:
            raise KernelError(f"decode_inputs: {name} is shorter than slots")
    _check("decode_inputs", lib().tib_decode_inputs(_ptr(records), _ptr(slots), c_int(records.shape[0]), _ptr(token_ids),
                                                    _ptr(positions), c_int(n), _stream()))


def attention_mma_supports(head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernels are built for this head size and group size."""
    return bool(lib().tib_attention_mma_supports(c_int(head_dim), c_int(group)))


def _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim):
    _need(q, "q", torch.bfloat16), _need(pool, "pool", torch.bfloat16), _need(out, "out", torch.bfloat16)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"attention: pool shape {tuple(pool.shape)} does not fit")
    if q.numel() != out.numel() or q.numel() % (heads * head_dim):
        raise KernelError("attention: q / out do not fit the head counts")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("attention: entry arrays are shorter than n_entries")


def prefill_attention(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                      kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                      max_q_len: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      skip_single: bool = False) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tensor cores (bf16)."""
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    _check("prefill_attention", lib().tib_prefill_attention(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(int(skip_single)), _stream()))
    return out


def decode_split(n_entries: int, heads: int, kv_heads: int, max_kv_len: int, target_blocks: int = 148) -> tuple[int, int]:
    """(num_splits, chunk) for a known longest context: about ``target_blocks`` blocks, two tiles a split at least."""
    group = heads // kv_heads
    blocks = max(1, n_entries * kv_heads * ((group + 15) // 16))
    tiles = max(1, -(-max_kv_len // 64))
    splits = max(1, min(-(-tiles // 2), -(-target_blocks // blocks)))
    per = -(-tiles // splits)
    return -(-tiles // per), per * 64


# What tib_plan_attention answers (csrc/block.cu), and what it may be allowed to use.
ATTENTION_NONE, ATTENTION_PREFILL_TCGEN05, ATTENTION_PREFILL_MMA, ATTENTION_DECODE_TMA_ROTATES, ATTENTION_DECODE_TMA, \
    ATTENTION_DECODE_CP_ASYNC, ATTENTION_SIMT = range(7)
ALLOW_PREFILL_TCGEN05, ALLOW_DECODE_ROTATES, ALLOW_DECODE_TMA = 1, 2, 4
PRODUCT_LIBRARY, PRODUCT_DECODE, PRODUCT_SWAPAB = 0, 1, 2


def plan_attention(head_dim: int, group: int, page_size: int, packed: bool, n_entries: int, n_single: int, n_multi: int,
                   allow: int) -> tuple[int, int]:
    """(kernel for the portions of prompts, kernel for the single tokens) of a bfloat16 step, as the CUDA library
    chooses them: the one place where that is decided, for the part-by-part sequence and the native block alike."""
    prefill, decode = c_int(0), c_int(0)
    _check("plan_attention", lib().tib_plan_attention(c_int(head_dim), c_int(group), c_int(page_size), c_int(int(packed)),
                                                      c_int(n_entries), c_int(n_single), c_int(n_multi), c_int(allow),
                                                      ctypes.byref(prefill), ctypes.byref(decode)))
    return prefill.value, decode.value


def plan_product(rows: int, n: int, k: int, kn: bool, few_rows: int, features: int, splits: int, swiglu: bool,
                 aligned: bool) -> int:
    """The kernel a bf16 product of ``rows`` rows goes to (PRODUCT_*), chosen in the same place for both ways of
    running a block."""
    return int(lib().tib_plan_product(c_int(rows), c_int(n), c_int(k), c_int(int(kn)), c_int(few_rows), c_int(features),
                                      c_int(splits), c_int(int(swiglu)), c_int(int(aligned))))


def decode_num_splits(n_entries: int, heads: int, kv_heads: int, max_kv_len: int | None = None,
                      target_blocks: int = 256, slots: int = 296) -> int:
    """How many parts the grid provides for each request's context when the kernel sizes the parts itself.

    Measured on the B200 at 3,072 tokens of context (32 heads, 8 kv heads of 128): the kernel is fastest
    with about 256 blocks in all, just under the two per SM that fit (batch 1: 16 parts, 2: 8 to 16, 4: 8,
    8: 4, 16: 2, 32 and up: 1); more than 16 parts cost more in the merge than they gain, except where the
    context may be long (``max_kv_len`` above 8,192: one request at 32,768 tokens streams at 3.1 TB/s in 16
    parts, 128 blocks), where up to 32 are provided.  The TMA kernel uses only as many of them as the
    request's own context has stretches of 192 keys.

    ``slots``: the blocks that run at once (two on each of 148 SMs).  A batch a little larger than that would run
    one full round and a nearly empty second one; cut in two or three parts its blocks are more and shorter rounds
    (2,100 tokens of context, 38 / 44 / 48 / 52 requests: 95 / 99 / 101 / 103 us in one part, 85 / 91 / 95 / 105 in
    three, 89 / 94 / 95 / 99 in two; from 56 requests on, and past two rounds, one part is fastest again)."""
    group = heads // kv_heads
    blocks = max(1, n_entries * kv_heads * ((group + 15) // 16))
    if slots < blocks < 2 * slots:
        last_round = blocks / slots - 1            # how full the second round would be
        if last_round <= 0.2:
            return 3
        if last_round <= 0.45:
            return 2
    most = 32 if max_kv_len is not None and max_kv_len > 8192 else 16
    return max(1, min(most, target_blocks // blocks))


def decode_attention(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                     kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                     heads: int, kv_heads: int, head_dim: int, scale: float, max_kv_len: int, window: int = 0,
                     scratch: torch.Tensor | None = None, num_splits: int | None = None,
                     chunk: int | None = None, kernel: str = "auto", error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of single tokens over the paged cache, the context split over blocks (bf16).

    ``kernel``: "tma" (keys and values copied by the TMA unit; see ``decode_attention_tma_supports``),
    "cp_async" (every key row fetched by its own address; any page size), or "auto": the first where
    it takes the shape.

    Entries that bring more than one token are skipped.  ``max_kv_len`` bounds the longest context
    (keys 0 .. position) of the batch when ``num_splits`` and ``chunk`` are given (by default the kernel
    cuts each request's own context into equal parts); ``scratch`` (fp32, at least n_entries * heads * num_splits *
    (head_dim + 2) elements) holds the partial results when there is more than one split.
    """
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    if num_splits is None or chunk is None:
        # each request's own context is cut into num_splits equal parts by the kernel (chunk 0)
        num_splits, chunk = decode_num_splits(n_entries, heads, kv_heads, max_kv_len), 0
    elif chunk != 0 and num_splits * chunk < max_kv_len:
        raise KernelError("decode_attention: num_splits * chunk does not cover the longest context")
    scratch_o = scratch_ml = None
    if num_splits > 1:
        need = n_entries * heads * num_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError("decode_attention: scratch is too small")
        scratch_o = scratch
        scratch_ml = scratch[n_entries * heads * num_splits * head_dim:]
    if kernel not in ("auto", "tma", "cp_async"):
        raise KernelError(f"decode_attention: no kernel {kernel!r}")
    packed = pool.stride(0) == 2 * kv_heads * pool.shape[3] * head_dim
    tma = plan_attention(head_dim, heads // kv_heads, pool.shape[3], packed, n_entries, n_entries, 0,
                         0 if kernel == "cp_async" else ALLOW_DECODE_TMA)[1] == ATTENTION_DECODE_TMA
    if kernel == "tma" and not tma:
        raise KernelError("decode_attention: the TMA kernel does not take this shape "
                          f"(head_dim {head_dim}, group {heads // kv_heads}, pages of {pool.shape[3]}, packed={packed})")
    if tma:
        _check("decode_attention_tma", lib().tib_decode_attention_tma(
            _ptr(q), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
            _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
            c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
            c_int(num_splits), c_int(chunk), _ptr(_split_counters(q.device, n_entries * kv_heads) if num_splits > 1 else None),
            _ptr(error_word), _stream()))
        return out
    _check("decode_attention", lib().tib_decode_attention(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(num_splits), c_int(chunk), _stream()))
    return out


def decode_attention_rope(qkv: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                          kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                          heads: int, kv_heads: int, head_dim: int, scale: float, max_kv_len: int, inv_freq: torch.Tensor,
                          *, rot_dim: int | None = None, interleaved: bool = False, window: int = 0,
                          scratch: torch.Tensor | None = None, num_splits: int | None = None,
                          error_word: torch.Tensor | None = None) -> torch.Tensor:
    """A step of single tokens straight from the rows of the qkv product: the TMA decode kernel rotates the queries,
    rotates each token's key and writes it and the value into the token's page, then attends
    (:func:`rope_append` followed by :func:`decode_attention`, in one kernel and bit for bit).  Every entry must bring
    one token; needs a shape the TMA kernel takes (``decode_attention_tma_supports``)."""
    _need(qkv, "qkv", torch.bfloat16), _need(pool, "pool", torch.bfloat16), _need(out, "out", torch.bfloat16)
    _need(inv_freq, "inv_freq", torch.float32)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    rot = head_dim if rot_dim is None else rot_dim
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"attention: pool shape {tuple(pool.shape)} does not fit")
    if qkv.dim() != 2 or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim or out.shape != (qkv.shape[0], heads * head_dim):
        raise KernelError("decode_attention_rope: qkv / out do not fit the head counts")
    if inv_freq.numel() != rot // 2:
        raise KernelError("decode_attention_rope: inv_freq has the wrong length")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("attention: entry arrays are shorter than n_entries")
    packed = pool.stride(0) == 2 * kv_heads * pool.shape[3] * head_dim
    if not (packed and decode_attention_tma_supports(head_dim, heads // kv_heads, pool.shape[3])):
        raise KernelError("decode_attention_rope: the TMA kernel does not take this shape")
    if num_splits is None:
        num_splits = decode_num_splits(n_entries, heads, kv_heads, max_kv_len)
    scratch_o = scratch_ml = None
    if num_splits > 1:
        need = n_entries * heads * num_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError("decode_attention: scratch is too small")
        scratch_o, scratch_ml = scratch, scratch[n_entries * heads * num_splits * head_dim:]
    _check("decode_attention_tma_rope", lib().tib_decode_attention_tma_rope(
        _ptr(qkv), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(num_splits), c_int(0), _ptr(_split_counters(qkv.device, n_entries * kv_heads) if num_splits > 1 else None),
        _ptr(error_word), _ptr(inv_freq), c_int(rot), c_int(int(interleaved)), _stream()))
    return out


_counters: dict[torch.device, torch.Tensor] = {}
_COUNTERS = 65536     # allocated once per device, outside any graph capture that may come later


def _split_counters(device: torch.device, n: int) -> torch.Tensor | None:
    """Zeroed ints in which the parts of a split context count themselves in (the kernel leaves them zero).
    One buffer per device: launches on one stream follow one another."""
    if n > _COUNTERS:
        return None            # (the kernel then merges with a second launch)
    have = _counters.get(device)
    if have is None:
        have = _counters[device] = torch.zeros(_COUNTERS, dtype=torch.int32, device=device)
    return have


def decode_attention_tma_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(lib().tib_decode_attention_tma_supports(c_int(head_dim), c_int(group), c_int(page_size)))


_blas_workspace: dict[int, torch.Tensor] = {}
BLAS_WORKSPACE_BYTES = 32 << 20


def library_gemm_ready(device: torch.device) -> None:
    """Make the cuBLAS handle of ``device`` and give it its workspace (once)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _blas_workspace:
        buffer = torch.empty(BLAS_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        with torch.cuda.device(index):
            status = lib().tib_blas_init(_ptr(buffer), ctypes.c_size_t(buffer.numel()))
        if status:
            raise KernelError(f"library_gemm: cuBLAS could not be set up (status {status})")
        _blas_workspace[index] = buffer


def library_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, w_kn: bool) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w^T by cuBLAS, called from the engine's own library: ``w`` is stored
    [N, K], or [K, N] when ``w_kn``.  The library's workspace is a buffer of this module, made at the first call on
    a device (make that call outside a stream capture)."""
    library_gemm_ready(x.device)
    m, k = x.shape
    n = w.shape[1] if w_kn else w.shape[0]
    if (w.shape[0] if w_kn else w.shape[1]) != k or out.shape != (m, n):
        raise KernelError(f"library_gemm: shapes {tuple(x.shape)}, {tuple(w.shape)} (kn={w_kn}), {tuple(out.shape)} do not fit")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("library_gemm: bf16 operands with unit inner stride are needed")
    status = lib().tib_blas_gemm(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
                                 c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(1 if w_kn else 0),
                                 c_int(_code(out.dtype)), _stream())
    if status:
        raise KernelError(f"library_gemm: status {status} (20000 + n: cuBLAS status n)")
    return out        # (a library kernel: not counted among this library's launches)


def gemm_tcgen05_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w[N, K]^T on tcgen05 tensor cores (TMA loads, TMEM accumulator)."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05", lib().tib_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                                  c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                                  c_int(_code(out.dtype)), _ptr(error_word), _stream()))
    return out


def gemm_tcgen05_2cta_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_2cta_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05_2cta(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w[N, K]^T on pairs of SMs (`tcgen05.mma.cta_group::2`, 256 x 256 tiles)."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05_2cta: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05_2cta: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05_2cta", lib().tib_gemm_tcgen05_2cta(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                                            c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                                            c_int(_code(out.dtype)), _ptr(error_word), _stream()))
    return out


def gemm_tcgen05_swapab_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_swapab_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05_swapab(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None,
                        splits: int = 0, w_kn: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] . w^T for M <= 64 on tcgen05 tensor cores with the operands swapped: w ([N, K], or
    [K, N] with ``w_kn``) is streamed by TMA as the 128-row operand, K is split over a thread-block cluster
    (``splits`` = 0: chosen by the library) and the partial tiles are summed through distributed shared memory."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05_swapab: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    m, k = x.shape
    k2, n = w.shape if w_kn else (w.shape[1], w.shape[0])
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05_swapab: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05_swapab", lib().tib_gemm_tcgen05_swapab(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)), c_int64(w.stride(0)),
        c_int64(out.stride(0)), c_int(int(w_kn)), c_int(_code(out.dtype)), c_int(splits), _ptr(error_word), _stream()))
    return out


DG_PLAIN, DG_SWIGLU = 0, 1


def gemm_decode_supports(m: int, n: int, k: int, features: int = 128, splits: int = 1, epilogue: int = DG_PLAIN) -> bool:
    return bool(lib().tib_gemm_decode_supports(c_int(m), c_int(n), c_int(k), c_int(features), c_int(splits), c_int(epilogue)))


def gemm_decode(x: torch.Tensor, w_kn: torch.Tensor, out: torch.Tensor, *, features: int = 128, splits: int = 1,
                epilogue: int = DG_PLAIN, stages: int = 0, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """The product of a decode step, out[M, N] = x[M, K] . w for M <= 64 with ``w_kn`` stored [K, N]: tiles of
    ``features`` (128 or 256) features streamed by TMA through a ring of ``stages`` stages (0: the kernel's default),
    K shared by ``splits`` blocks of a cluster.  With the SwiGLU
    epilogue ``w_kn`` holds gate and up columns interleaved and ``out`` is the activation [M, N / 2]."""
    for name, t in (("x", x), ("w_kn", w_kn)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_decode: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (k2, n) = x.shape, w_kn.shape
    if k != k2 or out.shape != (m, n // 2 if epilogue == DG_SWIGLU else n):
        raise KernelError(f"gemm_decode: shapes {tuple(x.shape)} x {tuple(w_kn.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_decode", lib().tib_gemm_decode(
        _ptr(x), _ptr(w_kn), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)), c_int64(w_kn.stride(0)),
        c_int64(out.stride(0)), c_int(_code(out.dtype)), c_int(features), c_int(splits), c_int(epilogue), c_int(stages),
        _ptr(error_word), _stream()))
    return out


def prefill_attention_tcgen05_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(lib().tib_prefill_attention_tcgen05_supports(c_int(head_dim), c_int(group), c_int(page_size)))


def prefill_attention_tcgen05(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                              kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                              max_q_len: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
                              skip_single: bool = False, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tcgen05 tensor cores (bf16): S and O in
    TMEM, Q / K / V tiles by TMA, softmax in fp32 by one thread per row."""
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    _check("prefill_attention_tcgen05", lib().tib_prefill_attention_tcgen05(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(q.numel() // (heads * head_dim)),
        c_int(heads), c_int(kv_heads), c_int(head_dim), c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]),
        c_int(window), c_float(scale), c_int(int(skip_single)), _ptr(error_word), _stream()))
    return out


# ---------------------------------------------------------------------------
# Row-wise pieces of blocks other than the pre-norm one (csrc/gated_ops.cu).  Operands may be float32 or bfloat16
# and may be column slices of a wider row (unit inner stride, any row stride).
def _rows_of(t: torch.Tensor, name: str, width: int | None = None) -> None:
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a 2-D CUDA tensor with unit inner stride")
    if width is not None and t.shape[1] != width:
        raise KernelError(f"{name} has {t.shape[1]} columns, wanted {width}")


def add_pair(residual: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None = None,
             copy: torch.Tensor | None = None) -> torch.Tensor:
    """residual += a + b in fp32 (``b`` may be None); ``copy``, if given, receives the new residual in its own type."""
    _need(residual, "residual", torch.float32)
    n, width = residual.shape
    _rows_of(a, "a", width)
    if b is not None:
        _rows_of(b, "b", width)
    if copy is not None:
        _need(copy, "copy")
        if copy.shape != residual.shape:
            raise KernelError("add_pair: copy and residual differ in shape")
    if a.shape[0] != n or (b is not None and b.shape[0] != n):
        raise KernelError("add_pair: row counts differ")
    _check("add_pair", lib().tib_add_pair(
        _ptr(residual), _ptr(a), c_int(_code(a.dtype)), c_int64(a.stride(0)), _ptr(b),
        c_int(_code(b.dtype) if b is not None else 0), c_int64(b.stride(0) if b is not None else 0), _ptr(copy),
        c_int(_code(copy.dtype) if copy is not None else 0), c_int(n), c_int(width), _stream()))
    return residual


def unit_norm_add(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """residual += y / sqrt(mean(y^2) + eps) * weight, statistics and sum in fp32."""
    _need(residual, "residual", torch.float32), _need(weight, "weight", torch.float32)
    n, width = residual.shape
    _rows_of(y, "y", width)
    if y.shape[0] != n or weight.numel() != width:
        raise KernelError("unit_norm_add: shapes do not fit")
    _check("unit_norm_add", lib().tib_unit_norm_add(_ptr(residual), _ptr(y), c_int(_code(y.dtype)), c_int64(y.stride(0)),
                                                    _ptr(weight), c_int(n), c_int(width), c_float(eps), _stream()))
    return residual


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, weight: torch.Tensor | None = None,
                 eps: float = 0.0, group: int = 1) -> torch.Tensor:
    """out = f(x) * sigmoid(gate) row by row; f is the RMS norm with ``weight`` when one is given, else the identity.
    ``group`` > 1: one gate per run of ``group`` columns (a head), ``gate`` then has width / group columns."""
    _need(out, "out")
    n, width = out.shape
    if group < 1 or width % group:
        raise KernelError("sigmoid_gate: the group does not divide the width")
    _rows_of(x, "x", width), _rows_of(gate, "gate", width // group)
    if weight is not None:
        _need(weight, "weight", torch.float32)
        if weight.numel() != width:
            raise KernelError("sigmoid_gate: weight has the wrong length")
    if x.shape[0] != n or gate.shape[0] != n:
        raise KernelError("sigmoid_gate: row counts differ")
    _check("sigmoid_gate", lib().tib_sigmoid_gate(
        _ptr(x), c_int(_code(x.dtype)), c_int64(x.stride(0)), _ptr(gate), c_int(_code(gate.dtype)), c_int64(gate.stride(0)),
        _ptr(weight), c_float(eps), _ptr(out), c_int(_code(out.dtype)), c_int(n), c_int(width), c_int(group), _stream()))
    return out


def gelu_gate_table(a: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, first: int, out: torch.Tensor) -> torch.Tensor:
    """out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], first + j]."""
    _need(out, "out"), _need(ids, "ids", torch.int32)
    n, width = out.shape
    _rows_of(a, "a", width), _rows_of(table, "table")
    if a.shape[0] != n or ids.numel() != n or first < 0 or first + width > table.shape[1]:
        raise KernelError("gelu_gate_table: shapes do not fit")
    _check("gelu_gate_table", lib().tib_gelu_gate_table(
        _ptr(a), c_int(_code(a.dtype)), c_int64(a.stride(0)), _ptr(ids), _ptr(table), c_int(_code(table.dtype)),
        c_int64(table.stride(0)), c_int(table.shape[0]), c_int(first), _ptr(out), c_int(_code(out.dtype)), c_int(n),
        c_int(width), _stream()))
    return out


def relu_squared(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(x, "x"), _need(out, "out")
    if x.numel() != out.numel():
        raise KernelError("relu_squared: sizes differ")
    _check("relu_squared", lib().tib_relu_squared(_ptr(x), c_int(_code(x.dtype)), _ptr(out), c_int(_code(out.dtype)),
                                                  c_int64(x.numel()), _stream()))
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor (fp32, in place)."""
    _need(x, "x", torch.float32)
    _check("scale", lib().tib_scale_f32(_ptr(x), c_float(factor), c_int64(x.numel()), _stream()))
    return x


def pair_rows(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = [x[t] ; y[t]] in out's type (x, y fp32)."""
    _need(x, "x", torch.float32), _need(y, "y", torch.float32), _need(out, "out")
    n, width = x.shape
    if y.shape != x.shape or out.shape != (n, 2 * width):
        raise KernelError("pair_rows: shapes do not fit")
    _check("pair_rows", lib().tib_pair_rows(_ptr(x), _ptr(y), _ptr(out), c_int(_code(out.dtype)), c_int(n), c_int(width), _stream()))
    return out


def add_vector(x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """x[t] += v for every row (fp32)."""
    _need(x, "x", torch.float32), _need(v, "v", torch.float32)
    if v.numel() != x.shape[1]:
        raise KernelError("add_vector: the vector has the wrong length")
    _check("add_vector", lib().tib_add_vector(_ptr(x), _ptr(v), c_int(x.shape[0]), c_int(x.shape[1]), _stream()))
    return x


# ---------------------------------------------------------------------------
def library_gemm_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, w_kn: bool) -> torch.Tensor:
    """out[:, b, :] = x[:, b, :] . w[b]^T for every b, by one cuBLAS call.  ``x``: [M, B, K] and ``out``: [M, B, N] are views
    with unit inner stride whose rows (M) and batches (B) lie at any strides; ``w``: [B, N, K], or [B, K, N] when ``w_kn``."""
    library_gemm_ready(x.device)
    m, batch, k = x.shape
    n = w.shape[2] if w_kn else w.shape[1]
    if w.shape[0] != batch or (w.shape[1] if w_kn else w.shape[2]) != k or out.shape != (m, batch, n):
        raise KernelError(f"library_gemm_batched: shapes {tuple(x.shape)}, {tuple(w.shape)} (kn={w_kn}), {tuple(out.shape)} do not fit")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(2) != 1 or w.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("library_gemm_batched: bf16 operands with unit inner stride are needed")
    status = lib().tib_blas_gemm_batched(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)), c_int64(w.stride(1)),
        c_int64(out.stride(0)), c_int64(x.stride(1)), c_int64(w.stride(0)), c_int64(out.stride(1)), c_int(batch),
        c_int(1 if w_kn else 0), c_int(_code(out.dtype)), _stream())
    if status:
        raise KernelError(f"library_gemm_batched: status {status} (20000 + n: cuBLAS status n)")
    return out


# ---------------------------------------------------------------------------
def linear_attention_chunk(key_dim: int, value_dim: int) -> int:
    """Tokens per chunk of the decayed linear attention kernel for these head sizes (0: they do not fit an SM)."""
    return int(lib().tib_linear_attention_chunk(c_int(key_dim), c_int(value_dim)))


def linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, state: torch.Tensor,
                     powers: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, n_entries: int, heads: int,
                     key_dim: int, value_dim: int, *, silu: bool) -> torch.Tensor:
    """o_t = S_t^T q_t with S_t = decay * S_(t-1) + k_t v_t^T per head, over the ragged batch; ``state``
    [slots, heads, key_dim, value_dim] (fp32) is read and left updated; ``powers`` [heads, chunk + 1] holds decay^m."""
    for name, t, width in (("q", q, heads * key_dim), ("k", k, heads * key_dim), ("v", v, heads * value_dim)):
        _rows_of(t, name, width)
        if t.dtype != q.dtype:
            raise KernelError("linear_attention: q, k and v differ in type")
    _need(out, "out", torch.float32), _need(state, "state", torch.float32), _need(powers, "powers", torch.float32)
    _need(q_start, "q_start", torch.int32), _need(slots, "slots", torch.int32)
    chunk = powers.shape[1] - 1
    if out.shape != (q.shape[0], heads * value_dim) or tuple(state.shape[1:]) != (heads, key_dim, value_dim) or powers.shape[0] != heads:
        raise KernelError("linear_attention: out, state or powers do not fit the head sizes")
    if q_start.numel() < n_entries + 1 or slots.numel() < n_entries:
        raise KernelError("linear_attention: entry arrays are shorter than n_entries")
    _check("linear_attention", lib().tib_linear_attention(
        _ptr(q), _ptr(k), _ptr(v), c_int64(q.stride(0)), c_int64(k.stride(0)), c_int64(v.stride(0)), _ptr(out), _ptr(state),
        _ptr(powers), _ptr(q_start), _ptr(slots), c_int(n_entries), c_int(heads), c_int(key_dim), c_int(value_dim),
        c_int(chunk), c_int(1 if silu else 0), c_int(_code(q.dtype)), _stream()))
    return out


# ---------------------------------------------------------------------------
def latent_append(dkv: torch.Tensor, q: torch.Tensor, folded: torch.Tensor, keys: torch.Tensor | None,
                  positions: torch.Tensor, token_slot: torch.Tensor | None, block_table: torch.Tensor | None,
                  norm_weight: torch.Tensor, eps: float, inv_freq: torch.Tensor, heads: int, dim: int, rank: int, rot: int,
                  error_word: torch.Tensor | None = None, half_pairs: bool = False) -> None:
    """Norm the latent, rotate the shared key part and store both in the tokens' pages (``keys``: [pages, 1, page_size,
    rank + rot], or None to store nothing); rotate every head's query part into ``folded[..., rank:]``.  The rotary pairs
    are (2i, 2i + 1), or with ``half_pairs`` (i, i + len(inv_freq)), over the first 2 * len(inv_freq) rotated elements."""
    _rows_of(dkv, "dkv", rank + rot), _rows_of(q, "q", heads * (dim + rot))
    _need(folded, "folded", torch.float32), _need(positions, "positions", torch.int32)
    _need(norm_weight, "norm_weight", torch.float32), _need(inv_freq, "inv_freq", torch.float32)
    n = dkv.shape[0]
    if q.dtype != dkv.dtype or q.shape[0] != n or folded.shape != (n, heads, rank + rot) or norm_weight.numel() != rank:
        raise KernelError("latent_append: shapes or types do not fit")
    page_size = page_stride = num_pages = table_stride = 0
    if keys is not None:
        if token_slot is None or block_table is None:
            raise KernelError("latent_append: token_slot and block_table are needed to write the cache")
        _need(token_slot, "token_slot", torch.int32), _need(block_table, "block_table", torch.int32)
        if keys.dtype != dkv.dtype or keys.dim() != 4 or keys.shape[1] != 1 or keys.shape[3] != rank + rot or keys.stride(3) != 1 \
                or keys.stride(2) != rank + rot:
            raise KernelError(f"latent_append: pages of shape {tuple(keys.shape)} do not fit")
        num_pages, page_size, page_stride, table_stride = keys.shape[0], keys.shape[2], keys.stride(0), block_table.stride(0)
    _check("latent_append", lib().tib_latent_append(
        _ptr(dkv), c_int64(dkv.stride(0)), _ptr(q), c_int64(q.stride(0)), _ptr(keys), _ptr(folded), _ptr(positions),
        _ptr(token_slot), _ptr(block_table), c_int(table_stride), _ptr(norm_weight), c_float(eps), _ptr(inv_freq),
        c_int(inv_freq.numel()), c_int(n), c_int(heads), c_int(dim), c_int(rank), c_int(rot), c_int(page_size),
        c_int64(page_stride), c_int(num_pages), c_int(int(half_pairs)), _ptr(error_word), c_int(_code(dkv.dtype)), _stream()))


def latent_attention(folded: torch.Tensor, keys: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor, kv_start: torch.Tensor,
                     slots: torch.Tensor, block_table: torch.Tensor, n_entries: int, max_q_len: int, heads: int, rank: int,
                     rot: int, scale: float, error_word: torch.Tensor | None = None, max_kv_len: int = 0,
                     force_simt: bool = False) -> torch.Tensor:
    """Causal attention of folded queries [tokens, heads, rank + rot] (fp32) over paged latent rows; the value of a
    key is its first ``rank`` elements.  ``out``: [tokens, heads, rank] fp32.  A step of single tokens only
    (``max_q_len`` 1) that names the longest context (``max_kv_len``) cuts every context into runs that go to blocks of
    their own and are merged by a second kernel."""
    _need(folded, "folded", torch.float32), _need(out, "out", torch.float32)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    n = folded.shape[0]
    if folded.shape != (n, heads, rank + rot) or out.shape != (n, heads, rank):
        raise KernelError("latent_attention: folded / out do not fit the sizes")
    if keys.dim() != 4 or keys.shape[1] != 1 or keys.shape[3] != rank + rot or keys.stride(3) != 1 or keys.stride(2) != rank + rot:
        raise KernelError(f"latent_attention: pages of shape {tuple(keys.shape)} do not fit")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("latent_attention: entry arrays are shorter than n_entries")
    splits, partial = 1, None
    if max_q_len == 1 and max_kv_len > 0 and n == n_entries:
        splits = int(lib().tib_latent_attention_splits(c_int(n_entries), c_int(heads), c_int(max_kv_len)))
        if splits > 1:
            partial = torch.empty((n, heads, splits, 2 + rank), dtype=torch.float32, device=folded.device)
    _check("latent_attention", lib().tib_latent_attention(
        _ptr(folded), _ptr(keys), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(rank), c_int(rot),
        c_int(keys.shape[2]), c_int64(keys.stride(0)), c_int(keys.shape[0]), c_float(scale), _ptr(partial), c_int(splits),
        c_int(max_kv_len), c_int(int(force_simt)), _ptr(error_word), c_int(_code(keys.dtype)), _stream()))
    if partial is not None:
        count_launches(1)
    return out


# ---------------------------------------------------------------------------
MOE_ACT = {"none": 0, "relu2": 1, "silu": 2, "glu_clamp": 3, "swiglu": 4}
MOE_GATED = ("glu_clamp", "swiglu")      # activations over (gate, up) row pairs: half as many columns leave


def router_logits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, e] = x[t] . w[e] in fp32, for a few rows ``w`` (fp32): every sum in an order fixed by k alone."""
    _rows_of(x, "x"), _need(w, "w", torch.float32), _rows_of(out, "out")
    if out.dtype != torch.float32 or w.dim() != 2 or x.shape[1] != w.shape[1] or out.shape != (x.shape[0], w.shape[0]):
        raise KernelError("router_logits: shapes or types do not fit")
    _check("router_logits", lib().tib_router_logits(_ptr(x), c_int(_code(x.dtype)), c_int64(x.stride(0)), _ptr(w), _ptr(out),
                                                    c_int64(out.stride(0)), c_int(x.shape[0]), c_int(w.shape[0]), c_int(x.shape[1]),
                                                    _stream()))
    return out


def moe_route(logits: torch.Tensor, experts: int, top: int, ids: torch.Tensor, weights: torch.Tensor, *,
              sigmoid_scores: bool = False, normalize: bool = True, norm_eps: float = 0.0,
              correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1) -> None:
    """From fp32 router logits (the first ``experts`` columns of ``logits``): the ``top`` best experts of every token and
    their weights.  ``correction`` [experts] is added to the scores for the choice only (the weights are made from the
    scores themselves); with ``groups`` > 1 the outputs are cut into that many equal runs of adjacent ones, every run is
    ranked by the best corrected score in it, and only members of the ``keep`` best runs are eligible."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1 or logits.shape[1] < experts:
        raise KernelError("moe_route: logits must be 2-D fp32 with unit inner stride and at least `experts` columns")
    _need(ids, "ids", torch.int32), _need(weights, "weights", torch.float32)
    n = logits.shape[0]
    if ids.shape != (n, top) or weights.shape != (n, top):
        raise KernelError("moe_route: ids / weights must be [tokens, top]")
    if correction is not None:
        _need(correction, "correction", torch.float32)
        if correction.numel() != experts:
            raise KernelError("moe_route: correction must hold one number per expert")
    if groups <= 1:
        groups = keep = 1
    _check("moe_route", lib().tib_moe_route(_ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(experts), c_int(top),
                                            c_int(int(sigmoid_scores)), c_int(int(normalize)), c_float(norm_eps),
                                            _ptr(correction), c_int(groups), c_int(keep), _ptr(ids), _ptr(weights), _stream()))


def moe_group(ids: torch.Tensor, experts: int, offsets: torch.Tensor, order: torch.Tensor, place: torch.Tensor) -> None:
    """Sort the (token, choice) pairs by expert on the device: offsets [experts + 1], order[sorted] = pair, place[pair] = sorted."""
    for name, t in (("ids", ids), ("offsets", offsets), ("order", order), ("place", place)):
        _need(t, name, torch.int32)
    pairs = ids.numel()
    if offsets.numel() != experts + 1 or order.numel() != pairs or place.numel() != pairs:
        raise KernelError("moe_group: array lengths do not fit")
    _check("moe_group", lib().tib_moe_group(_ptr(ids), c_int(pairs), c_int(experts), _ptr(offsets), _ptr(order), _ptr(place), _stream()))


def moe_expert_product(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor, top: int,
                       *, x_by_pair: bool, act: str = "none", limit: float = 0.0, alpha: float = 1.0,
                       row_scale: torch.Tensor | None = None) -> torch.Tensor:
    """y[s] = act(row_scale[pair of s] * (x[source of s] . w[expert of s]^T)) for the sorted rows s; ``w``: [experts, N, K];
    ``x_by_pair``: the source of sorted row s is token order[s] // top, else row s itself.  ``act="glu_clamp"``: the rows
    of ``w`` are (gate i, up i) pairs and y has N / 2 columns: g * sigmoid(alpha g) * (u + 1) with g = min(g, limit),
    u = clamp(u, -limit, limit); ``act="swiglu"``: silu(g) * u over the same pairs.  ``row_scale``: one fp32 factor per
    (token, choice) pair, or None."""
    _rows_of(x, "x"), _need(w, "w"), _rows_of(y, "y")
    experts, n, k = w.shape
    pairs = order.numel()
    if x.shape[1] != k or y.shape != (pairs, n // 2 if act in MOE_GATED else n) or offsets.numel() != experts + 1:
        raise KernelError("moe_expert_product: shapes do not fit")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32)
        if row_scale.numel() != pairs:
            raise KernelError("moe_expert_product: row_scale must hold one factor per pair")
    _check("moe_expert_product", lib().tib_moe_expert_product(
        _ptr(x), c_int(_code(x.dtype)), c_int64(x.stride(0)), _ptr(w), c_int(_code(w.dtype)), _ptr(y), c_int(_code(y.dtype)),
        c_int64(y.stride(0)), _ptr(offsets), _ptr(order), c_int(pairs), c_int(experts), c_int(top), c_int(int(x_by_pair)),
        c_int(n), c_int(k), c_int(MOE_ACT[act]), c_float(limit), c_float(alpha), _ptr(row_scale), _stream()))
    return y


def moe_combine(y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor,
                shared: torch.Tensor | None = None, gate: torch.Tensor | None = None, *, ids: torch.Tensor | None = None,
                identity_from: int = 0, x: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[place[t, k]] (+ sigmoid(gate[t]) * shared[t]); ``gate``: one fp32 logit per token
    (a column view is fine); ``weights`` None: every weight is 1 (``place`` then is [tokens, top]).  With ``ids`` [tokens,
    top], a choice whose id is ``identity_from`` or above stands for no expert: it adds weights[t, k] * x[t], the experts'
    input rows ``x`` (of ``out``'s type)."""
    _need(y, "y", torch.float32), _need(place, "place", torch.int32), _need(out, "out")
    n, width = out.shape
    if weights is not None:
        _need(weights, "weights", torch.float32)
        top = weights.shape[1]
    else:
        top = place.numel() // max(n, 1)
    if y.shape[1] != width or (weights is not None and weights.shape[0] != n) or place.numel() != n * top:
        raise KernelError("moe_combine: shapes do not fit")
    if shared is not None:
        _need(shared, "shared")
        if shared.shape != out.shape:
            raise KernelError("moe_combine: shared rows do not fit")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.shape[0] != n:
            raise KernelError("moe_combine: gate must hold one fp32 logit per token")
        ld_gate = gate.stride(0)
    ldx = 0
    if ids is not None:
        _need(ids, "ids", torch.int32)
        if x is None or ids.numel() != n * top:
            raise KernelError("moe_combine: choices that hand the input through need ids [tokens, top] and the input rows")
        _rows_of(x, "x", width)
        if x.dtype != out.dtype or x.shape[0] != n:
            raise KernelError("moe_combine: the input rows must have the output's type and row count")
        ldx = x.stride(0)
    _check("moe_combine", lib().tib_moe_combine(
        _ptr(y), _ptr(place), _ptr(weights), c_int(top), _ptr(shared), c_int(_code(shared.dtype) if shared is not None else 0),
        _ptr(gate), c_int64(ld_gate), _ptr(out), c_int(_code(out.dtype)), c_int(n), c_int(width), _ptr(ids),
        c_int(identity_from), _ptr(x if ids is not None else None), c_int64(ldx), _stream()))
    return out


def glu_clamp(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out[t, i] = g * sigmoid(alpha g) * (u + 1) with g = min(gate_up[t, 2i], limit), u = clamp(gate_up[t, 2i + 1], -limit, limit)."""
    _need(gate_up, "gate_up"), _need(out, "out")
    n, width = out.shape
    if gate_up.shape != (n, 2 * width):
        raise KernelError("glu_clamp: gate_up must be [rows, 2 * width]")
    _check("glu_clamp", lib().tib_glu_clamp(_ptr(gate_up), c_int(_code(gate_up.dtype)), _ptr(out), c_int(_code(out.dtype)), c_int(n),
                                            c_int(width), c_float(limit), c_float(alpha), _stream()))
    return out


# ---------------------------------------------------------------------------
# Layer norm with weight and bias, the tails of sublayers and layers built on it (csrc/layernorm.cu).
def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out: torch.Tensor,
              rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[i] = LN(x[rows[i]] or x[i]) in fp32; x: fp32 or bf16 rows (any row stride), out: [n, width] in its own type."""
    _rows_of(x, "x"), _need(weight, "weight", torch.float32), _need(bias, "bias", torch.float32), _need(out, "out")
    width = x.shape[1]
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if out.shape != (n, width) or weight.numel() != width or bias.numel() != width:
        raise KernelError("layernorm: shapes do not fit")
    _check("layernorm", lib().tib_layernorm(_ptr(x), c_int(_code(x.dtype)), c_int64(x.stride(0)), _ptr(rows), _ptr(weight), _ptr(bias),
                                            c_float(eps), _ptr(out), c_int(_code(out.dtype)), c_int(n), c_int(width), _stream()))
    return out


def layernorm_tail(residual: torch.Tensor, eps: float, *, y: torch.Tensor | None = None, y_norm: tuple | None = None,
                   history: torch.Tensor | None = None, coef: torch.Tensor | None = None, count: int = 0,
                   out: torch.Tensor | None = None, out_norm: tuple | None = None) -> None:
    """What follows a sublayer, in one launch: ``residual += LN(y; *y_norm)`` (if ``y``; with ``y_norm`` None: ``residual
    += y``); then, if ``history``
    ([depth, n, width] fp32 whose slice ``count - 1`` is ``residual``), ``history[count] = sum_j coef[j] * history[j]``
    over j < count; then, if ``out``, ``out = LN(the row at hand; *out_norm)``.  Norms are (weight, bias) in fp32."""
    _need(residual, "residual", torch.float32)
    n, width = residual.shape
    wa = ba = wb = bb = None
    if y is not None:
        _rows_of(y, "y", width)
        if y.shape[0] != n:
            raise KernelError("layernorm_tail: y does not fit")
        if y_norm is not None:
            wa, ba = y_norm
            if wa.numel() != width or ba.numel() != width or wa.dtype != torch.float32 or ba.dtype != torch.float32:
                raise KernelError("layernorm_tail: the norm of y does not fit")
    slice_elems = 0
    if history is not None:
        _need(history, "history", torch.float32), _need(coef, "coef", torch.float32)
        if (history.dim() != 3 or history.shape[1:] != (n, width) or not 1 <= count < history.shape[0] or coef.numel() < count
                or history[count - 1].data_ptr() != residual.data_ptr()):
            raise KernelError("layernorm_tail: the history does not fit")
        slice_elems = history.stride(0)
    if out is not None:
        _need(out, "out")
        wb, bb = out_norm
        if out.shape != (n, width) or wb.numel() != width or bb.numel() != width or wb.dtype != torch.float32 or bb.dtype != torch.float32:
            raise KernelError("layernorm_tail: out or its norm do not fit")
    _check("layernorm_tail", lib().tib_layernorm_tail(
        _ptr(y), c_int(_code(y.dtype) if y is not None else 0), c_int64(y.stride(0) if y is not None else 0), _ptr(wa), _ptr(ba),
        _ptr(residual), _ptr(history), c_int64(slice_elems), _ptr(coef), c_int(count), _ptr(wb), _ptr(bb), _ptr(out),
        c_int(_code(out.dtype) if out is not None else 0), c_int(n), c_int(width), c_float(eps), _stream()))


# ---------------------------------------------------------------------------
# Attention with sigmoid weights (csrc/sigmoid_attention.cu).
def qk_norm_append(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, keys: torch.Tensor | None,
                   values: torch.Tensor | None, positions: torch.Tensor, token_slot: torch.Tensor | None,
                   block_table: torch.Tensor | None, inv_freq: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                   *, rot_dim: int, interleaved: bool = False, eps: float = -1.0, error_word: torch.Tensor | None = None,
                   q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None, temp_coef: float = 0.0,
                   temp_every: int = 0) -> torch.Tensor:
    """Rotate part of every q and k head of the fused projection ``proj`` (columns q_off.., k_off.., v_off..), divide each
    head by its root mean square (``eps`` < 0: not), write q to ``q_out`` and k, v into their pages (``keys`` /
    ``values``: [pages, kv_heads, page_size, dim / vdim] views of one layer's pages).  ``keys`` None: only q.
    ``q_weight`` / ``k_weight`` [dim] multiply every normed q / k head; ``temp_every`` > 0 multiplies every q by
    1 + temp_coef * ln(floor((position + 1) / temp_every) + 1).  ``inv_freq`` may be None when ``rot_dim`` is 0."""
    _rows_of(proj, "proj"), _need(q_out, "q_out", proj.dtype), _need(positions, "positions", torch.int32)
    n = proj.shape[0]
    if q_out.shape != (n, heads * dim):
        raise KernelError("qk_norm_append: q_out must be [tokens, heads * dim]")
    write = keys is not None
    page_size = page_stride = num_pages = table_stride = 0
    if write:
        if keys.dtype != proj.dtype or values is None or values.dtype != proj.dtype:
            raise KernelError("qk_norm_append: the pages must have the projection's type")
        if keys.shape[1:] != (kv_heads, keys.shape[2], dim) or values.shape[1:] != (kv_heads, keys.shape[2], vdim) \
                or keys.stride(0) != values.stride(0) or not keys[0].is_contiguous() or not values[0].is_contiguous():
            raise KernelError("qk_norm_append: keys / values are not one layer's pages")
        _need(token_slot, "token_slot", torch.int32), _need(block_table, "block_table", torch.int32)
        num_pages, page_size, page_stride, table_stride = keys.shape[0], keys.shape[2], keys.stride(0), block_table.stride(0)
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != dim or not t.is_contiguous() or not t.is_cuda):
            raise KernelError(f"qk_norm_append: {name} must be {dim} fp32 numbers")
    _check("qk_norm_append", lib().tib_qk_norm_append(
        _ptr(proj), c_int64(proj.stride(0)), c_int(q_off), c_int(k_off if write else -1), c_int(v_off), _ptr(q_out),
        _ptr(keys), _ptr(values), _ptr(positions), _ptr(token_slot if write else None), _ptr(block_table if write else None),
        c_int(table_stride), _ptr(inv_freq), c_int(n), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(rot_dim),
        c_int(int(interleaved)), c_float(eps), c_int(page_size), c_int64(page_stride), c_int(num_pages), _ptr(q_weight),
        _ptr(k_weight), c_float(temp_coef), c_int(temp_every), _ptr(error_word), c_int(_code(proj.dtype)), _stream()))
    return q_out


def sigmoid_attention(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                      kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int, max_q_len: int,
                      heads: int, kv_heads: int, *, scale: float, chunk: int = 0, window: int = 0,
                      head_bias: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                      error_word: torch.Tensor | None = None, force_simt: bool = False, max_kv_len: int | None = None,
                      splits: int | None = None) -> torch.Tensor:
    """out[i] = sigmoid(gate[i]) * sum over visible j of sigmoid(q_i . k_j * scale + head_bias) * v_j, per head; visible:
    j <= i, in i's chunk of ``chunk`` positions (0: no chunks) and within ``window`` (0: none).  ``gate``: [tokens, heads]
    logits (a column slice is fine) or None.  bfloat16 with head sizes that are multiples of 8 up to 128 runs on the tensor
    cores, everything else (and ``force_simt``) on the CUDA-core kernel.  In a step of single tokens on the tensor cores the
    keys of each context are shared out over ``splits`` blocks (None: enough to fill the GPU, from ``max_kv_len``, a bound
    on the longest context) whose sums are added in a fixed order by a second small kernel."""
    _need(q, "q"), _need(out, "out", q.dtype)
    dim, vdim, page_size = keys.shape[3], values.shape[3], keys.shape[2]
    n = q.shape[0]
    if q.shape != (n, heads * dim) or out.shape != (n, heads * vdim) or keys.dtype != q.dtype or values.dtype != q.dtype:
        raise KernelError("sigmoid_attention: shapes or types do not fit")
    if keys.stride(0) != values.stride(0) or not keys[0].is_contiguous() or not values[0].is_contiguous():
        raise KernelError("sigmoid_attention: keys / values are not one layer's pages")
    if head_bias is not None:
        _need(head_bias, "head_bias", torch.float32)
    if gate is not None:
        _rows_of(gate, "gate", heads)
    partial = None
    if (max_q_len == 1 and q.dtype == torch.bfloat16 and not force_simt
            and lib().tib_sigmoid_attention_takes_mma(c_int(dim), c_int(vdim))):
        if splits is None:
            seen = min(x for x in (chunk or None, window or None, max_kv_len, 1 << 30) if x)
            tiles = -(-seen // 64) + 1
            blocks = n_entries * kv_heads * -(-(heads // kv_heads) // 64)
            splits = min(tiles, max(1, 2 * 148 // blocks))      # (two blocks fit an SM: one wave)
        if splits > 1:
            partial = torch.empty((splits, n_entries, heads * vdim), dtype=torch.float32, device=q.device)
            count_launches(1)
    splits = splits if partial is not None else 0
    _check("sigmoid_attention", lib().tib_sigmoid_attention(
        _ptr(q), _ptr(keys), _ptr(values), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim),
        c_int(page_size), c_int64(keys.stride(0)), c_int(keys.shape[0]), c_int(chunk), c_int(window), c_float(scale),
        _ptr(head_bias), _ptr(gate), c_int(_code(gate.dtype) if gate is not None else 0),
        c_int64(gate.stride(0) if gate is not None else 0), _ptr(error_word), c_int(_code(q.dtype)), c_int(int(force_simt)),
        c_int(splits), _ptr(partial), _stream()))
    return out


# ---------------------------------------------------------------------------
GATED_RECURRENCE_RUN = 64       # tokens of a portion that one thread scans; longer portions are scanned run by run, side by side


def gated_recurrence(proj: torch.Tensor, z_off: int, u_off: int, g_off: int, bias_z: torch.Tensor | None,
                     bias_u: torch.Tensor | None, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
                     out: torch.Tensor, n_entries: int, max_q_len: int, run_len: int = GATED_RECURRENCE_RUN) -> torch.Tensor:
    """The element-wise gated recurrence S = (1 - z) S + z c over each entry's tokens, from and to ``state[slot]`` (fp32);
    z = sigmoid(proj[:, z_off..] + bias_z), c from proj[:, u_off..] + bias_u, out = S * silu(proj[:, g_off..]) (g_off < 0: S)."""
    _rows_of(proj, "proj"), _need(state, "state", torch.float32), _need(out, "out")
    width = out.shape[1]
    if out.shape[0] != proj.shape[0] or state.dim() != 2 or state.shape[1] != width:
        raise KernelError("gated_recurrence: shapes do not fit")
    for b in (bias_z, bias_u):
        if b is not None:
            _need(b, "bias", torch.float32)
    runs = -(-max_q_len // run_len)
    run_a = run_b = None
    if runs > 1:
        scratch = torch.empty((2, n_entries, runs, width), dtype=torch.float32, device=out.device)
        run_a, run_b = scratch[0], scratch[1]
    status = lib().tib_gated_recurrence(
        _ptr(proj), c_int(_code(proj.dtype)), c_int64(proj.stride(0)), c_int(z_off), c_int(u_off), c_int(g_off), _ptr(bias_z),
        _ptr(bias_u), _ptr(state), _ptr(q_start), _ptr(slots), _ptr(out), c_int(_code(out.dtype)), _ptr(run_a), _ptr(run_b),
        c_int(n_entries), c_int(max_q_len), c_int(width), c_int(run_len), _stream())
    _check("gated_recurrence", status)
    if runs > 1:
        count_launches(1)
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) (fp32, in place)."""
    _need(x, "x", torch.float32)
    if not cap > 0:
        raise KernelError("softcap: the cap is positive")
    _check("softcap", lib().tib_softcap_f32(_ptr(x), c_float(cap), c_int64(x.numel()), _stream()))
    return x


# ---------------------------------------------------------------------------
# The state-space mixer (csrc/state_space.cu).
def short_conv(rows: torch.Tensor, col: int, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor, state_off: int,
               q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, n_entries: int, max_q_len: int, *,
               silu: bool = True) -> torch.Tensor:
    """out[t, c] = act(bias[c] + sum_k weight[c, k] * rows[t - taps + 1 + k, col + c]), causal within each entry of the
    ragged batch; the taps - 1 inputs before an entry's first token come from ``state[slot, state_off:]`` (laid out
    [taps - 1, channels]), where the kernel then leaves the entry's last taps - 1 inputs.  act: silu, or the identity."""
    _rows_of(rows, "rows"), _need(weight, "weight", torch.float32), _need(state, "state", torch.float32), _need(out, "out")
    channels, taps = weight.shape
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if (out.shape != (rows.shape[0], channels) or col < 0 or col + channels > rows.shape[1] or state.dim() != 2
            or state_off < 0 or state_off + (taps - 1) * channels > state.shape[1] or (bias is not None and bias.numel() != channels)):
        raise KernelError("short_conv: shapes do not fit")
    _check("short_conv", lib().tib_short_conv(
        _ptr(rows), c_int(_code(rows.dtype)), c_int64(rows.stride(0)), c_int(col), _ptr(weight), _ptr(bias), _ptr(state),
        c_int64(state.stride(0)), c_int64(state_off), _ptr(q_start), _ptr(slots), _ptr(out), c_int(_code(out.dtype)), c_int(channels),
        c_int(taps), c_int(int(silu)), c_int(n_entries), c_int(max_q_len), _stream()))
    return out


def ssd_scan_max_state() -> int:
    return int(lib().tib_ssd_scan_max_state())


_scan_run: int | None = None


def ssd_scan_run() -> int:
    """How many tokens the scan walks in one piece when it cuts long portions."""
    global _scan_run
    if _scan_run is None:
        _scan_run = int(lib().tib_ssd_scan_run())
    return _scan_run


def ssd_scan(xbc: torch.Tensor, dt_rows: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, y: torch.Tensor, n_entries: int, *, heads: int,
             groups: int, state_dim: int, head_dim: int, max_q_len: int | None = None) -> torch.Tensor:
    """The recurrence S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t per head over the ragged batch;
    ``xbc`` rows hold [x | B | C]; ``dt_rows[:, dt_col + h]`` the raw step size of head h; S is the first
    heads * state_dim * head_dim floats of ``state[slot]`` (fp32), read at the start and left at the end.
    ``max_q_len``: the longest entry of the step; when it exceeds one run of the kernel, portions are cut into runs that
    are walked side by side (scratch for the runs' states is allocated here); None: every portion in one piece."""
    _rows_of(xbc, "xbc", heads * head_dim + 2 * groups * state_dim), _rows_of(dt_rows, "dt_rows")
    _need(state, "state", torch.float32), _need(y, "y", torch.float32)
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _need(t, name, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"ssd_scan: {name} has the wrong length")
    if (y.shape != (xbc.shape[0], heads * head_dim) or dt_rows.shape[0] != xbc.shape[0] or dt_col < 0
            or dt_col + heads > dt_rows.shape[1] or state.dim() != 2 or state.shape[1] < heads * state_dim * head_dim):
        raise KernelError("ssd_scan: shapes do not fit")
    n_tokens = xbc.shape[0]
    run_state = run_decay = None
    capacity = 0
    if max_q_len is not None and max_q_len > ssd_scan_run():
        capacity = n_tokens // ssd_scan_run() + n_entries
        run_state = torch.empty((capacity, heads * state_dim * head_dim), dtype=torch.float32, device=xbc.device)
        run_decay = torch.empty((capacity, heads), dtype=torch.float32, device=xbc.device)
    _check("ssd_scan", lib().tib_ssd_scan(
        _ptr(xbc), c_int(_code(xbc.dtype)), c_int64(xbc.stride(0)), _ptr(dt_rows), c_int(_code(dt_rows.dtype)),
        c_int64(dt_rows.stride(0)), c_int(dt_col), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), c_int64(state.stride(0)),
        _ptr(q_start), _ptr(slots), _ptr(y), c_int(heads), c_int(groups), c_int(state_dim), c_int(head_dim), c_int(n_entries),
        c_int(n_tokens), c_int(n_tokens if max_q_len is None else max_q_len), _ptr(run_state), _ptr(run_decay), c_int64(capacity),
        _stream()))
    return y


def gated_group_norm(y: torch.Tensor, z_rows: torch.Tensor, z_col: int, weight: torch.Tensor, eps: float, out: torch.Tensor,
                     parts: int) -> torch.Tensor:
    """out = v / sqrt(mean(v^2) + eps) * weight with v = y * silu(z) and the mean taken over each of ``parts`` equal runs
    of the row; y fp32, z = ``z_rows[:, z_col : z_col + width]``."""
    _need(y, "y", torch.float32), _rows_of(z_rows, "z_rows"), _need(weight, "weight", torch.float32), _need(out, "out")
    n, width = y.shape
    if out.shape != y.shape or weight.numel() != width or z_rows.shape[0] != n or z_col < 0 or z_col + width > z_rows.shape[1]:
        raise KernelError("gated_group_norm: shapes do not fit")
    _check("gated_group_norm", lib().tib_gated_group_norm(
        _ptr(y), _ptr(z_rows), c_int(_code(z_rows.dtype)), c_int64(z_rows.stride(0)), c_int(z_col), _ptr(weight), c_float(eps),
        _ptr(out), c_int(_code(out.dtype)), c_int(n), c_int(width), c_int(parts), _stream()))
    return out


# ---------------------------------------------------------------------------
# Attention over a window and pooled blocks (csrc/pooled_window_attention.cu).
def _pages(keys: torch.Tensor, values: torch.Tensor, kv_heads: int, dim: int, vdim: int, name: str) -> tuple[int, int, int]:
    """(num_pages, page_size, page_stride) of one layer's [pages, kv_heads, page_size, dim / vdim] views."""
    if (keys.shape[1:] != (kv_heads, keys.shape[2], dim) or values.shape[1:] != (kv_heads, keys.shape[2], vdim)
            or keys.stride(0) != values.stride(0) or not keys[0].is_contiguous() or not values[0].is_contiguous()
            or keys.dtype != values.dtype):
        raise KernelError(f"{name}: keys / values are not one layer's pages")
    return keys.shape[0], keys.shape[2], keys.stride(0)


def rotary_kv_append(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, keys: torch.Tensor,
                     values: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor, block_table: torch.Tensor,
                     freq: torch.Tensor, value_freq: torch.Tensor | None, heads: int, kv_heads: int, dim: int, vdim: int, *,
                     rot_dim: int, amplitude: float = 1.0, q_bias: torch.Tensor | None = None, k_bias: torch.Tensor | None = None,
                     v_bias: torch.Tensor | None = None, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Add the biases, rotate the first ``rot_dim`` elements of every q and k head of the fused projection ``proj`` (pairs i,
    i + rot_dim / 2, cos and sin times ``amplitude``), turn every v head over its whole width by ``value_freq`` (None: not),
    write q to ``q_out`` and k, v into their pages."""
    _rows_of(proj, "proj"), _need(q_out, "q_out", proj.dtype), _need(positions, "positions", torch.int32)
    _need(token_slot, "token_slot", torch.int32), _need(block_table, "block_table", torch.int32), _need(freq, "freq", torch.float32)
    n = proj.shape[0]
    if q_out.shape != (n, heads * dim) or keys.dtype != proj.dtype or freq.numel() * 2 != rot_dim:
        raise KernelError("rotary_kv_append: shapes or types do not fit")
    for t, width in ((q_bias, heads * dim), (k_bias, kv_heads * dim), (v_bias, kv_heads * vdim)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous()):
            raise KernelError("rotary_kv_append: a bias does not fit")
    if value_freq is not None and (value_freq.dtype != torch.float32 or value_freq.numel() * 2 != vdim):
        raise KernelError("rotary_kv_append: value_freq does not fit")
    num_pages, page_size, page_stride = _pages(keys, values, kv_heads, dim, vdim, "rotary_kv_append")
    _check("rotary_kv_append", lib().tib_rotary_kv_append(
        _ptr(proj), c_int64(proj.stride(0)), c_int(q_off), c_int(k_off), c_int(v_off), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
        _ptr(q_out), _ptr(keys), _ptr(values), _ptr(positions), _ptr(token_slot), _ptr(block_table), c_int(block_table.stride(0)),
        _ptr(freq), _ptr(value_freq), c_float(amplitude), c_int(n), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim),
        c_int(rot_dim), c_int(page_size), c_int64(page_stride), c_int(num_pages), _ptr(error_word), c_int(_code(proj.dtype)), _stream()))
    return q_out


def pool_blocks(keys: torch.Tensor, values: torch.Tensor, block_table: torch.Tensor, block_keys: torch.Tensor,
                block_values: torch.Tensor, block_block_table: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor,
                pool: int, *, error_word: torch.Tensor | None = None) -> None:
    """For every token of the step that completes a block of ``pool`` positions, the mean of the block's cached keys and of
    its cached values goes into entry position // pool of the strided pages ``block_keys`` / ``block_values``."""
    kv_heads, dim, vdim = keys.shape[1], keys.shape[3], values.shape[3]
    num_pages, page_size, page_stride = _pages(keys, values, kv_heads, dim, vdim, "pool_blocks")
    b_pages, b_page_size, b_stride = _pages(block_keys, block_values, kv_heads, dim, vdim, "pool_blocks")
    if block_keys.dtype != keys.dtype:
        raise KernelError("pool_blocks: the two caches differ in type")
    _need(positions, "positions", torch.int32), _need(token_slot, "token_slot", torch.int32)
    _check("pool_blocks", lib().tib_pool_blocks(
        _ptr(keys), _ptr(values), _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), c_int64(page_stride),
        c_int(num_pages), _ptr(block_keys), _ptr(block_values), _ptr(block_block_table), c_int(block_block_table.stride(0)),
        c_int(b_page_size), c_int64(b_stride), c_int(b_pages), _ptr(positions), _ptr(token_slot), c_int(positions.numel()),
        c_int(kv_heads), c_int(dim), c_int(vdim), c_int(pool), _ptr(error_word), c_int(_code(keys.dtype)), _stream()))


def pooled_window_attention(q: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor, kv_start: torch.Tensor, slots: torch.Tensor,
                            keys: torch.Tensor, values: torch.Tensor, block_table: torch.Tensor, block_keys: torch.Tensor | None,
                            block_values: torch.Tensor | None, block_block_table: torch.Tensor | None, n_entries: int,
                            max_q_len: int, heads: int, kv_heads: int, *, window: int, pool: int, scale: float,
                            temp: torch.Tensor | None = None, sink: torch.Tensor | None = None,
                            value_freq: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                            error_word: torch.Tensor | None = None, force_simt: bool = False,
                            rel_bias: torch.Tensor | None = None, max_kv_len: int = 0, splits: int | None = None) -> torch.Tensor:
    """Per head, out[i] = sigmoid(gate[i]) * turn_back_i(sum_j w_ij v_j + sum_b w_ib V_b): softmax weights over the tokens j
    with 0 <= i - j < window and the blocks b of ``pool`` positions with b * pool + pool - 1 <= i - window (their means K_b,
    V_b from the strided pages), scores q . k * scale * temp[h], exp(sink[h]) added to the denominator; turn_back undoes at
    position i the rotation the values were cached with (``value_freq``; None: none).  ``pool`` 0: the window alone.
    ``rel_bias`` [heads, span] fp32: rel_bias[h, min(i - j, span - 1)] is added to the score of token j (as it is: neither
    ``scale`` nor ``temp`` multiplies it).  A step of single tokens only on the tensor cores (no turned values, no gate) that
    names the longest context (``max_kv_len``) shares every context's visible keys out over ``splits`` blocks (None: enough
    to fill the GPU) whose sums a second small kernel adds in a fixed order.
    bfloat16 steps run on the tensor cores when the head sizes are multiples of 8 up to 128, unless ``force_simt``."""
    _need(q, "q"), _need(out, "out", q.dtype)
    dim, vdim = keys.shape[3], values.shape[3]
    n = q.shape[0]
    if q.shape != (n, heads * dim) or out.shape != (n, heads * vdim) or keys.dtype != q.dtype:
        raise KernelError("pooled_window_attention: shapes or types do not fit")
    num_pages, page_size, page_stride = _pages(keys, values, kv_heads, dim, vdim, "pooled_window_attention")
    b_pages = b_page_size = b_stride = b_table_stride = 0
    if pool > 0:
        if block_keys is None or block_values is None or block_block_table is None or block_keys.dtype != q.dtype:
            raise KernelError("pooled_window_attention: blocks need their pages")
        b_pages, b_page_size, b_stride = _pages(block_keys, block_values, kv_heads, dim, vdim, "pooled_window_attention")
        b_table_stride = block_block_table.stride(0)
    for name, t in (("temp", temp), ("sink", sink)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous()):
            raise KernelError(f"pooled_window_attention: {name} does not fit")
    if value_freq is not None and (value_freq.dtype != torch.float32 or value_freq.numel() * 2 != vdim):
        raise KernelError("pooled_window_attention: value_freq does not fit")
    ld_gate = 0
    if gate is not None:
        _rows_of(gate, "gate", heads * vdim)
        ld_gate = gate.stride(0)
    if rel_bias is not None:
        _need(rel_bias, "rel_bias", torch.float32)
        if rel_bias.dim() != 2 or rel_bias.shape[0] != heads or rel_bias.shape[1] < 1:
            raise KernelError("pooled_window_attention: rel_bias must be [heads, span]")
    partial, n_splits = None, 1
    if (max_q_len == 1 and n == n_entries and max_kv_len > 0 and q.dtype == torch.bfloat16 and not force_simt
            and value_freq is None and gate is None and dim % 8 == 0 and vdim % 8 == 0 and dim <= 128 and vdim <= 128
            and heads // kv_heads <= 16):
        n_splits = splits if splits is not None else int(lib().tib_pooled_window_attention_splits(
            c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(min(window, max_kv_len) + (max_kv_len // pool if pool else 0))))
        if n_splits > 1:
            floats = int(lib().tib_pooled_window_attention_part_floats(c_int(vdim)))
            partial = torch.empty((n_splits, n, heads, floats), dtype=torch.float32, device=q.device)
            count_launches(1)
        else:
            n_splits = 1
    _check("pooled_window_attention", lib().tib_pooled_window_attention(
        _ptr(q), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(keys), _ptr(values), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), c_int64(page_stride), c_int(num_pages),
        _ptr(block_keys if pool > 0 else None), _ptr(block_values if pool > 0 else None),
        _ptr(block_block_table if pool > 0 else None), c_int(b_table_stride), c_int(b_page_size), c_int64(b_stride), c_int(b_pages),
        c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(window), c_int(pool),
        c_float(scale), _ptr(temp), _ptr(sink), _ptr(value_freq), _ptr(gate), c_int(_code(gate.dtype) if gate is not None else 0),
        c_int64(ld_gate), _ptr(rel_bias), c_int(rel_bias.shape[1] if rel_bias is not None else 0), _ptr(partial),
        c_int(n_splits), c_int(n), _ptr(error_word), c_int(_code(q.dtype)), c_int(int(force_simt)), _stream()))
    return out


# ---------------------------------------------------------------------------
# A residual in several streams, and the tanh norm (csrc/hyper_streams.cu).
def hyper_step(streams: torch.Tensor, *, y: torch.Tensor | None = None, mix: torch.Tensor | None = None,
               out_weights: torch.Tensor | None = None, in_weights: torch.Tensor | None = None, out: torch.Tensor | None = None,
               rows: torch.Tensor | None = None, tanh_norm: tuple[float, torch.Tensor, torch.Tensor] | None = None
               ) -> torch.Tensor | None:
    """On streams [S, tokens, width] (fp32), in one launch: with ``y`` the write x_t <- sum_s mix[s, t] x_s + out_weights[t] y
    (every stream from the values before the write), then with ``in_weights`` the read u = sum_s in_weights[s] x_s into ``out``: as fp32
    sums, or with ``tanh_norm`` = (alpha, weight, bias) as tanh(alpha u) * weight + bias in ``out``'s type.  With ``rows``
    (int32 token rows) only those rows are read, ``out`` has one row per index and nothing is stored."""
    if not streams.is_cuda or streams.dtype != torch.float32 or streams.dim() != 3:
        raise KernelError("hyper_step: streams must be a CUDA fp32 tensor [S, tokens, width]")
    count, n, width = streams.shape
    if streams.stride(2) != 1 or streams.stride(1) != width:
        raise KernelError("hyper_step: every stream must be contiguous rows (the streams may lie apart)")
    if y is not None:
        _rows_of(y, "y", width)
        if y.shape[0] != n or mix is None or out_weights is None:
            raise KernelError("hyper_step: a write needs y [tokens, width], mix and out_weights")
        _need(mix, "mix", torch.float32), _need(out_weights, "out_weights", torch.float32)
        if mix.shape != (count, count) or out_weights.numel() != count:
            raise KernelError("hyper_step: mix must be [S, S] and out_weights [S]")
    n_out = n
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    norm, alpha, weight, bias = 0, 0.0, None, None
    if in_weights is not None:
        _need(in_weights, "in_weights", torch.float32)
        if out is None or in_weights.numel() != count:
            raise KernelError("hyper_step: a read needs in_weights [S] and out")
        _need(out, "out")
        if out.shape != (n_out, width):
            raise KernelError(f"hyper_step: out is {tuple(out.shape)}, wanted {(n_out, width)}")
        if tanh_norm is not None:
            alpha, weight, bias = tanh_norm
            _need(weight, "weight", torch.float32), _need(bias, "bias", torch.float32)
            if weight.numel() != width or bias.numel() != width:
                raise KernelError("hyper_step: the norm's weight and bias do not fit the width")
            norm = 1
        elif out.dtype != torch.float32:
            raise KernelError("hyper_step: sums without a norm leave in fp32")
    elif rows is not None:
        raise KernelError("hyper_step: rows only make sense with a read")
    _check("hyper_step", lib().tib_hyper_step(
        _ptr(streams), c_int64(streams.stride(0)), c_int(count), c_int(n_out), c_int(width), _ptr(y),
        c_int(_code(y.dtype) if y is not None else 0), c_int64(y.stride(0) if y is not None else 0), _ptr(mix),
        _ptr(out_weights), _ptr(in_weights), _ptr(rows), c_int(norm), c_float(alpha), _ptr(weight), _ptr(bias), _ptr(out),
        c_int(_code(out.dtype) if out is not None else 0), _stream()))
    return out
