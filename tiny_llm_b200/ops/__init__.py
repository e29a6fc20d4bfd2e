"""Python face of the sm_100a kernels.  Every op checks its tensors, picks the kernel for the
dtype and sizes, and launches it on torch's current stream through the C entry points of the
shared objects that `build.py` compiles from csrc/.  There is no other path: an op given a tensor
that is not on a CUDA device, or called where the kernels cannot be built, raises."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build
from .build import BuildError

F32, BF16 = 0, 1
OUT_SAME, OUT_F32, OUT_ACC = 0, 1, 2


class KernelError(RuntimeError):
    """A kernel refused its arguments (a size it is not built for) or failed to launch."""


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # torch's current stream of the current device as a raw cudaStream_t (the private accessor is
    # an order of magnitude cheaper than building a Stream object for every launch)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's ops run on a CUDA device only; got a tensor on " + str(t.device))


launches = 0  # kernels launched through this module since import (each entry point launches one)
_pdl = True


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch: each kernel is launched so that its prologue (and, for the
    matrix products, its first weight tiles) may overlap the tail of the kernel before it."""
    global _pdl
    _pdl = bool(on)
    for lib in build._loaded.values():
        lib.tllm_set_pdl(1 if _pdl else 0)


_tape = None   # while a list: every launch is also noted there as (library, function, arguments), see begin_tape()


def _call(lib, fn, *args):
    """Calls one entry point of a compiled library (one kernel launch, or a few) and raises its message if it refuses."""
    global launches
    if fn(*args) != 0:
        raise KernelError(lib.tllm_last_error().decode())
    launches += 1
    if _tape is not None:
        _tape.append((lib, fn, args))


def begin_tape() -> None:
    """From here to end_tape() the launches are noted as they are made: the compiled functions with the very argument
    objects they got.  A step whose launches depend on nothing but what the caller knows (the sizes of the step and the
    addresses of buffers that stay where they are) can be run again from such a tape without walking the model's
    Python code: the step's tables are read by the kernels from device memory, as in a captured graph."""
    global _tape
    _tape = []


def end_tape():
    global _tape
    tape, _tape = _tape, None
    return tape


def replay_tape(tape) -> None:
    global launches
    for lib, fn, args in tape:
        if fn(*args) != 0:
            raise KernelError(lib.tllm_last_error().decode())
    launches += len(tape)


def knobs():
    """The module's switches that decide which kernels a step launches; a tape or graph holds for one setting of them."""
    return (force_generic, split_k, cluster_mask, attention_tc, decode_wide_ctas, decode_cluster_merge, qkv_fused_rows,
            linear_skinny, generic_attention_split, split_mixed_attention, min_gru_segment, linear_attention_segment, moe_mma, moe_wide_tiles, moe_tc_rows_per_expert, window_attention_tc, window_attention_splits, attention_maps_tc, attention_maps_decode_pairs, attention_maps_splits, attention_talk_tc, attention_talk_splits, attention_talk_stages, _pdl)


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def trace_dump():
    """The timeline notes of every loaded library since the last call (needs a TLLM_TRACE=1 build):
    a list of (t_enter ns, t_ready ns, grid x, y, z, block x, library, marks), sorted by t_enter.  t_ready
    of a launch is when the kernel before it in the stream had finished; marks are up to four more
    moments a kernel noted itself (0: none)."""
    import struct
    out = []
    buf = ctypes.create_string_buffer(8192 * 64)
    for key, lib in build._loaded.items():
        if not hasattr(lib, "tllm_trace_dump"):
            continue
        n = lib.tllm_trace_dump(buf, 8192)
        for i in range(n):
            t0, t1, gx, gy, gz, bx, m0, m1, m2, m3 = struct.unpack_from("<QQIIIIQQQQ", buf, i * 64)
            out.append((t0, t1, gx, gy, gz, bx, key, (m0, m1, m2, m3)))
    return sorted(out)


# ----------------------------------------------------------------------------- elementwise


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
              scale: float = 1.0) -> None:
    """out[t, :] = table[tokens[t], :] * scale as float32 (the residual stream is 32-bit; the product is taken in
    32-bit); accumulate=True adds the rows into `out` instead (unscaled)."""
    _need_cuda(tokens, table, out)
    _i32(tokens, "tokens")
    t, h = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous() or table.shape[1] != h \
            or tokens.numel() != t:
        raise KernelError("embedding: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    if accumulate:
        if scale != 1.0:
            raise KernelError("embedding: rows that are added are not scaled")
        _call(lib, lib.tllm_embedding_add, _ptr(tokens), _ptr(table), _ptr(out), t, h, _code(table.dtype), _stream())
        return
    _call(lib, lib.tllm_embedding, _ptr(tokens), _ptr(table), _ptr(out), t, h, _code(table.dtype), ctypes.c_float(scale),
          _stream())


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = weight * x[rows[r], :] / sqrt(mean(x^2) + eps); x and weight are float32."""
    _need_cuda(x, weight, out, rows)
    _i32(rows, "rows")
    h = x.shape[1]
    n = out.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() or \
            not out.is_contiguous() or out.shape[1] != h or weight.numel() != h or \
            (rows is None and n != x.shape[0]) or (rows is not None and rows.numel() != n):
        raise KernelError("rms_norm: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rms_norm, _ptr(x), _ptr(weight), _ptr(out), _ptr(rows), n, h, ctypes.c_float(eps),
                                  _code(out.dtype), _stream())


def dyt_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = tanh(alpha * x[rows[r], :]) * weight + bias (Dynamic Tanh: no statistics); x, weight, bias and
    the one-element `alpha` are float32 on the device."""
    _need_cuda(x, weight, bias, alpha, out, rows)
    _i32(rows, "rows")
    h = x.shape[1]
    n = out.shape[0]
    if x.dtype != torch.float32 or any(v.dtype != torch.float32 for v in (weight, bias, alpha)) or \
            not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != h or weight.numel() != h or \
            bias.numel() != h or alpha.numel() != 1 or not weight.is_contiguous() or not bias.is_contiguous() or \
            (rows is None and n != x.shape[0]) or (rows is not None and rows.numel() != n):
        raise KernelError("dyt_norm: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_dyt_norm, _ptr(x), _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(out), _ptr(rows), n, h,
          _code(out.dtype), _stream())


def rope_pairs_kv_write(qkv: torch.Tensor, positions: torch.Tensor, freq: Optional[torch.Tensor], rot_dims: int,
                        num_q_rows: int, num_k_rows: int, num_v_rows: int, key_dim: int, value_dim: int,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Rows of `qkv`: num_q_rows query rows and num_k_rows key rows of key_dim values, then num_v_rows value rows of
    value_dim values.  The first rot_dims values of every query and key row are rotated pairwise (value 2i with
    2i + 1) by positions[t] * freq[i], in 32-bit; queries are rewritten in place, keys and values go to their pages
    (k_cache [pages, num_k_rows, page_size, key_dim], v_cache [pages, num_v_rows, page_size, value_dim])."""
    _need_cuda(qkv, positions, freq, k_cache, v_cache, slot_mapping)
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t, width = qkv.shape
    want = (num_q_rows + num_k_rows) * key_dim + num_v_rows * value_dim
    if width != want or qkv.stride(1) != 1:
        raise KernelError(f"rope_pairs_kv_write: rows of {width} values, expected {want}")
    if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or \
            k_cache.shape[1] != num_k_rows or k_cache.shape[3] != key_dim or k_cache.stride(3) != 1 or \
            k_cache.stride(2) != key_dim or v_cache.shape[1] != num_v_rows or v_cache.shape[3] != value_dim or \
            v_cache.stride(3) != 1 or v_cache.stride(2) != value_dim or k_cache.shape[2] != v_cache.shape[2]:
        raise KernelError("rope_pairs_kv_write: cache layout does not fit")
    if rot_dims and (freq is None or freq.dtype != torch.float32 or not freq.is_contiguous() or freq.numel() * 2 != rot_dims):
        raise KernelError("rope_pairs_kv_write: the frequency table does not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rope_pairs_kv_write, _ptr(qkv), _ptr(positions), _ptr(freq if rot_dims else None), rot_dims, t,
          num_q_rows, num_k_rows, num_v_rows, key_dim, value_dim, qkv.stride(0), _ptr(k_cache), _ptr(v_cache),
          _ptr(slot_mapping), k_cache.shape[2], ctypes.c_longlong(k_cache.stride(0)), ctypes.c_longlong(k_cache.stride(1)),
          ctypes.c_longlong(v_cache.stride(0)), ctypes.c_longlong(v_cache.stride(1)), _code(qkv.dtype), _stream())


def diff_combine(maps_out: torch.Tensor, lq1: torch.Tensor, lk1: torch.Tensor, lq2: torch.Tensor, lk2: torch.Tensor,
                 diff: float, eps: float, out: torch.Tensor) -> None:
    """maps_out: float32 [T, heads, 2, vd], the outputs a1, a2 of a head's two score maps.  With
    lam = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff:  o = a1 - lam * a2;  out[T, heads * vd] =
    o / sqrt(mean(o^2) + eps) * (1 - diff), all in 32-bit."""
    _need_cuda(maps_out, lq1, lk1, lq2, lk2, out)
    t, heads, two, vd = maps_out.shape
    kd = lq1.numel()
    if two != 2 or maps_out.dtype != torch.float32 or not maps_out.is_contiguous() or out.shape != (t, heads * vd) or \
            not out.is_contiguous() or any(v.dtype != torch.float32 or v.numel() != kd or not v.is_contiguous()
                                           for v in (lq1, lk1, lq2, lk2)):
        raise KernelError("diff_combine: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_diff_combine, _ptr(maps_out), _ptr(lq1), _ptr(lk1), _ptr(lq2), _ptr(lk2), kd,
          ctypes.c_float(diff), ctypes.c_float(eps), _ptr(out), ctypes.c_longlong(t * heads), vd, _code(out.dtype), _stream())


# Portions of at least this many tokens run the minGRU recurrence in segments (two kernels, every segment a thread
# per channel) instead of one thread per channel walking the whole portion; 0 turns the segments off.  The 32-bit
# path always walks serially: its results do not depend on how a sequence was cut into steps, to the bit.
min_gru_segment = int(os.environ.get("TLLM_MINGRU_SEGMENT", "32"))


def min_gru_scan(zug: torch.Tensor, bias_z: torch.Tensor, bias_u: torch.Tensor, state: torch.Tensor,
                 batch, out: torch.Tensor, workspace=None) -> None:
    """The minGRU recurrence over the step's tokens.  zug [T, 3 * width]: the projections [z | u | g];
    S_t = (1 - z_t) S_(t-1) + z_t c_t with z_t = sigmoid(z + bias_z), c_t = u + bias_u + 1/2 where that is >= 0 and
    sigmoid(u + bias_u) below; out[t] = S_t * silu(g).  state [slots, width] float32 holds S per request
    (batch.slots names each request's row) and is carried from step to step."""
    _need_cuda(zug, bias_z, bias_u, state, out)
    t, w3 = zug.shape
    width = w3 // 3
    if w3 != 3 * width or zug.stride(1) != 1 or out.shape != (t, width) or not out.is_contiguous() or \
            out.dtype != zug.dtype or state.dtype != torch.float32 or not state.is_contiguous() or \
            state.shape[1] != width or any(b.dtype != torch.float32 or b.numel() != width or not b.is_contiguous()
                                           for b in (bias_z, bias_u)):
        raise KernelError("min_gru_scan: shapes or dtypes do not fit")
    seg, summary = 0, None
    if zug.dtype == torch.bfloat16 and workspace is not None and min_gru_segment > 0 and \
            batch.max_q_len >= 2 * min_gru_segment:
        seg = min_gru_segment
        segs = -(-batch.max_q_len // seg)
        summary = workspace.get("min_gru_summary", (batch.num_requests * (2 * segs + 1) * width,), torch.float32)
    lib = build.load_library("recurrence")
    _call(lib, lib.tllm_min_gru_scan, _ptr(zug), zug.stride(0), _ptr(bias_z), _ptr(bias_u), _ptr(state),
          _ptr(batch.slots), _ptr(batch.cu_q), _ptr(out), width, batch.num_requests, batch.max_q_len, seg,
          _ptr(summary), _code(zug.dtype), _stream())


GLU_ACTS = {"silu": 0, "relu": 1}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int, consume: bool = False, act: str = "silu") -> None:
    """out[m, g*block + j] = act(gate_up[m, 2*g*block + j]) * gate_up[m, 2*g*block + block + j], act = silu or relu.
    `gate_up` is of out's dtype or float32 (a product's 32-bit sums).  consume=True: `gate_up` is a float32
    accumulation buffer (split-K sums) and is handed back zeroed."""
    _need_cuda(gate_up, out)
    m, inter = out.shape
    if gate_up.shape != (m, 2 * inter) or not gate_up.is_contiguous() or not out.is_contiguous() or \
            (consume and gate_up.dtype != torch.float32) or (not consume and gate_up.dtype not in (out.dtype, torch.float32)):
        raise KernelError("silu_mul: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    if act not in GLU_ACTS:
        raise KernelError(f"silu_mul: unknown activation {act!r} (known: {', '.join(GLU_ACTS)})")
    _call(lib, lib.tllm_silu_mul, _ptr(gate_up), _ptr(out), m, inter, block, _code(gate_up.dtype), _code(out.dtype),
                                  1 if consume else 0, GLU_ACTS[act], _stream())


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], rot_dim: int, num_heads: int, num_kv_heads: int, head_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  slot_mapping: Optional[torch.Tensor], src: Optional[torch.Tensor] = None) -> None:
    """Rotates the queries of `qkv` in place; rotates the keys and writes keys and values into the
    pages at slot_mapping (None: the row holds queries only and nothing is written).
    `src`: float32 rows to read instead of `qkv` (a split-K accumulation buffer, handed back zeroed);
    the rotated queries still go to `qkv`."""
    _need_cuda(qkv, positions, cos, sin, k_cache, v_cache, slot_mapping, src)
    if src is not None and (src.dtype != torch.float32 or src.shape != qkv.shape or src.stride(1) != 1):
        raise KernelError("rope_kv_write: the float32 source must have the shape of qkv")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t, width = qkv.shape
    want = num_heads * head_dim + (0 if slot_mapping is None else 2 * num_kv_heads * head_dim)
    if width != want or qkv.stride(1) != 1:
        raise KernelError(f"rope_kv_write: rows of {width} values, expected {want}")
    page_size = page_stride = head_stride = 0
    if slot_mapping is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or k_cache.shape != v_cache.shape or \
                k_cache.stride() != v_cache.stride() or k_cache.stride(3) != 1 or k_cache.stride(2) != head_dim:
            raise KernelError("rope_kv_write: cache layout does not fit")
        page_size, page_stride, head_stride = k_cache.shape[2], k_cache.stride(0), k_cache.stride(1)
    if cos is not None and (cos.dtype != torch.float32 or not cos.is_contiguous() or cos.shape[1] * 2 != rot_dim):
        raise KernelError("rope_kv_write: rotary tables do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rope_kv_write,
        _ptr(qkv), _ptr(src), 0 if src is None else src.stride(0), _ptr(positions), _ptr(cos), _ptr(sin), rot_dim, t,
        num_heads, num_kv_heads, head_dim,
        qkv.stride(0), _ptr(k_cache if slot_mapping is not None else None),
        _ptr(v_cache if slot_mapping is not None else None), _ptr(slot_mapping), page_size,
        ctypes.c_longlong(page_stride), ctypes.c_longlong(head_stride), _code(qkv.dtype), _stream())


# ----------------------------------------------------------------------------- linear attention, windows, experts


def rms_norm_add(x: torch.Tensor, weight: torch.Tensor, eps: float, scale: float, resid: torch.Tensor,
                 clear: bool = True, copy: Optional[torch.Tensor] = None) -> None:
    """resid += scale * weight * x / sqrt(mean(x^2) + eps), row by row, all float32; clear=True hands `x` back zeroed
    (a branch buffer that products accumulate into).  `copy` (bfloat16, resid's shape): also receives the new rows
    rounded, for a branch that reads the stream itself."""
    _need_cuda(x, weight, resid, copy)
    if copy is not None and (copy.dtype != torch.bfloat16 or copy.shape != resid.shape or not copy.is_contiguous()):
        raise KernelError("rms_norm_add: the copy is a contiguous bfloat16 tensor of the stream's shape")
    if x.dtype != torch.float32 or resid.dtype != torch.float32 or weight.dtype != torch.float32 or x.shape != resid.shape \
            or not x.is_contiguous() or not resid.is_contiguous() or weight.numel() != x.shape[1]:
        raise KernelError("rms_norm_add: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rms_norm_add, _ptr(x), _ptr(weight), _ptr(resid), x.shape[0], x.shape[1], ctypes.c_float(eps),
          ctypes.c_float(scale), 1 if clear else 0, _ptr(copy), _stream())


# Portions of at least 64 tokens run the linear-attention recurrence in segments of at most this many tokens (bfloat16
# only: the 32-bit path always walks a request's tokens in order, so that its state has the same bits however it was
# cut); 0: never.
linear_attention_segment = int(os.environ.get("TLLM_LINEAR_ATTENTION_SEGMENT", "128"))


def linear_attention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, key_dim: int, value_dim: int,
                          state: torch.Tensor, batch, out: torch.Tensor, q_scale: float = 1.0, k_scale: float = 1.0,
                          head_decay: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                          gate_bias: Optional[torch.Tensor] = None, inv_tau: float = 1.0, workspace=None) -> None:
    """S_t = diag(a_t) S_(t-1) + (k_scale k_t) v_t^T, out_t = S_t^T (q_scale q_t) per head, over the step's tokens.
    q, k [T, heads * key_dim], v [T, heads * value_dim] (row slices of a projection are fine); out float32
    [T, heads * value_dim]; state float32 [slots, heads, key_dim, value_dim], carried from step to step.
    a_t is `head_decay[h]` (float32 [heads]) for every channel, or sigmoid(gate + gate_bias)^inv_tau per key
    channel with `gate` float32 [T, heads * key_dim]."""
    _need_cuda(q, k, v, state, out, head_decay, gate, gate_bias)
    t = q.shape[0]
    if q.shape != (t, heads * key_dim) or k.shape != q.shape or v.shape != (t, heads * value_dim) or \
            q.dtype != k.dtype or q.dtype != v.dtype or any(x.stride(1) != 1 for x in (q, k, v)) or \
            out.shape != (t, heads * value_dim) or out.dtype != torch.float32 or not out.is_contiguous() or \
            state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, key_dim, value_dim):
        raise KernelError("linear_attention_scan: shapes or dtypes do not fit")
    if (head_decay is None) == (gate is None):
        raise KernelError("linear_attention_scan: give a decay per head or a gate, not both")
    if head_decay is not None and (head_decay.dtype != torch.float32 or head_decay.numel() != heads):
        raise KernelError("linear_attention_scan: one float32 decay per head")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != q.shape or gate.stride(1) != 1 or gate_bias is None or
                             gate_bias.dtype != torch.float32 or gate_bias.numel() != heads * key_dim):
        raise KernelError("linear_attention_scan: the gate and its bias do not fit")
    seg, summary = 0, None
    if q.dtype == torch.bfloat16 and workspace is not None and linear_attention_segment > 0 and batch.max_q_len >= 64:
        # shorter portions are cut finer, so that there are segments enough to fill the SMs: a sixteenth of the longest
        # portion, at least 32 tokens, at most the switch's value
        seg = min(linear_attention_segment, max(32, (batch.max_q_len // 16) // 8 * 8))
        segs = -(-batch.max_q_len // seg)
        per = heads * (key_dim * value_dim + key_dim)
        summary = workspace.get("lin_attn_summary", (batch.num_requests * segs * per,), torch.float32)
    lib = build.load_library("linear_attention")
    _call(lib, lib.tllm_linear_attention_scan, _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0),
          _ptr(head_decay), _ptr(gate), 0 if gate is None else gate.stride(0), _ptr(gate_bias), ctypes.c_float(inv_tau),
          ctypes.c_float(q_scale), ctypes.c_float(k_scale), _ptr(state), _ptr(batch.slots), _ptr(batch.cu_q), _ptr(out),
          heads, key_dim, value_dim, batch.num_requests, batch.max_q_len, seg, _ptr(summary), _code(q.dtype), _stream())


def head_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate: torch.Tensor, heads: int, value_dim: int,
                   eps: float, out: torch.Tensor, act: str = "silu") -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]) per (token, head), act = silu or sigmoid; o float32
    [T, heads * value_dim], weight float32 [value_dim] or None, gate and out [T, heads * value_dim] in the engine's dtype."""
    _need_cuda(o, weight, gate, out)
    t = o.shape[0]
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape != (t, heads * value_dim) or gate.shape != o.shape or \
            gate.stride(1) != 1 or out.shape != o.shape or not out.is_contiguous() or out.dtype != gate.dtype or \
            (weight is not None and (weight.dtype != torch.float32 or weight.numel() != value_dim)):
        raise KernelError("head_norm_gate: shapes or dtypes do not fit")
    if act not in ("silu", "sigmoid"):
        raise KernelError(f"head_norm_gate: unknown gate activation {act!r} (known: silu, sigmoid)")
    lib = build.load_library("linear_attention")
    _call(lib, lib.tllm_head_norm_gate, _ptr(o), _ptr(weight), _ptr(gate), gate.stride(0), heads, value_dim,
          ctypes.c_float(eps), _ptr(out), ctypes.c_longlong(t * heads), _code(out.dtype), 1 if act == "sigmoid" else 0,
          _stream())


def _paged(name: str, c: torch.Tensor, rows: int, dim: int) -> None:
    if c.dim() != 4 or c.shape[1] != rows or c.shape[3] != dim or c.stride(3) != 1 or c.stride(2) != dim:
        raise KernelError(f"{name}: cache layout does not fit (wanted [pages, {rows}, page_size, {dim}])")


def rope_halves_kv_write(qkv: torch.Tensor, positions: torch.Tensor, freq_k: Optional[torch.Tensor], rot_dims: int,
                         freq_v: Optional[torch.Tensor], num_q_rows: int, num_k_rows: int, num_v_rows: int, key_dim: int,
                         value_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Rows of `qkv`: query rows and key rows of key_dim values, then value rows of value_dim values.  The first
    rot_dims values of every query and key row are rotated (value i with value i + rot_dims / 2) by
    positions[t] * freq_k[i]; with `freq_v` the value rows are rotated over their whole size (value m with
    m + value_dim / 2) by positions[t] * freq_v[m].  Queries are rewritten in place, keys and values go to their pages."""
    _need_cuda(qkv, positions, freq_k, freq_v, k_cache, v_cache, slot_mapping)
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t, width = qkv.shape
    if width != (num_q_rows + num_k_rows) * key_dim + num_v_rows * value_dim or qkv.stride(1) != 1:
        raise KernelError("rope_halves_kv_write: the rows of qkv do not fit")
    _paged("rope_halves_kv_write", k_cache, num_k_rows, key_dim)
    _paged("rope_halves_kv_write", v_cache, num_v_rows, value_dim)
    if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or k_cache.shape[2] != v_cache.shape[2]:
        raise KernelError("rope_halves_kv_write: cache dtype or page size does not fit")
    for f, n in ((freq_k if rot_dims else None, rot_dims), (freq_v, value_dim)):
        if f is not None and (f.dtype != torch.float32 or not f.is_contiguous() or f.numel() * 2 != n):
            raise KernelError("rope_halves_kv_write: a frequency table does not fit")
    lib = build.load_library("window_attention")
    _call(lib, lib.tllm_rope_halves_kv_write, _ptr(qkv), _ptr(positions), _ptr(freq_k if rot_dims else None), rot_dims,
          _ptr(freq_v), t, num_q_rows, num_k_rows, num_v_rows, key_dim, value_dim, qkv.stride(0), _ptr(k_cache), _ptr(v_cache),
          _ptr(slot_mapping), k_cache.shape[2], ctypes.c_longlong(k_cache.stride(0)), ctypes.c_longlong(k_cache.stride(1)),
          ctypes.c_longlong(v_cache.stride(0)), ctypes.c_longlong(v_cache.stride(1)), _code(qkv.dtype), _stream())


def pool_kv_blocks(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor, pool_k: torch.Tensor,
                   pool_v: torch.Tensor, pool_slots: torch.Tensor, batch, pool: int) -> None:
    """Every token of the step whose entry of `pool_slots` is not negative completes a block of `pool` positions: the
    means of the block's cached keys and values (32-bit sums in the order of the positions) are written to that row
    of pool_k / pool_v."""
    _need_cuda(k_cache, v_cache, block_table, pool_k, pool_v, pool_slots)
    _i32(block_table, "block_table")
    _i32(pool_slots, "pool_slots")
    nkv, kd, vd = k_cache.shape[1], k_cache.shape[3], v_cache.shape[3]
    for name, c, d in (("k", k_cache, kd), ("v", v_cache, vd), ("pool k", pool_k, kd), ("pool v", pool_v, vd)):
        _paged("pool_kv_blocks", c, nkv, d)
    if len({c.dtype for c in (k_cache, v_cache, pool_k, pool_v)}) != 1 or len({c.shape[2] for c in (k_cache, v_cache, pool_k, pool_v)}) != 1:
        raise KernelError("pool_kv_blocks: the caches differ in dtype or page size")
    lib = build.load_library("window_attention")
    ll = ctypes.c_longlong
    _call(lib, lib.tllm_pool_kv_blocks, _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(pool_k),
          _ptr(pool_v), _ptr(pool_slots), _ptr(batch.positions), _ptr(batch.token_request), batch.num_tokens, nkv, pool, kd, vd,
          k_cache.shape[2], ll(k_cache.stride(0)), ll(k_cache.stride(1)), ll(v_cache.stride(0)), ll(v_cache.stride(1)),
          ll(pool_k.stride(0)), ll(pool_k.stride(1)), ll(pool_v.stride(0)), ll(pool_v.stride(1)), _code(k_cache.dtype), _stream())


class _WinArgs(ctypes.Structure):
    _fields_ = [("qkv", ctypes.c_void_p), ("row_stride", ctypes.c_int), ("nh", ctypes.c_int), ("nkv", ctypes.c_int),
                ("kd", ctypes.c_int), ("vd", ctypes.c_int), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("table", ctypes.c_void_p), ("max_blocks", ctypes.c_int),
                ("k_page_stride", ctypes.c_longlong), ("k_head_stride", ctypes.c_longlong),
                ("v_page_stride", ctypes.c_longlong), ("v_head_stride", ctypes.c_longlong),
                ("pk", ctypes.c_void_p), ("pv", ctypes.c_void_p), ("ptable", ctypes.c_void_p), ("pmax_blocks", ctypes.c_int),
                ("pk_page_stride", ctypes.c_longlong), ("pk_head_stride", ctypes.c_longlong),
                ("pv_page_stride", ctypes.c_longlong), ("pv_head_stride", ctypes.c_longlong),
                ("page_size", ctypes.c_int), ("positions", ctypes.c_void_p), ("token_request", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("scale", ctypes.c_float), ("cap", ctypes.c_float), ("head_bias", ctypes.c_void_p),
                ("window", ctypes.c_int), ("pool", ctypes.c_int), ("fv", ctypes.c_void_p), ("n_tokens", ctypes.c_int)]


# bfloat16 window attention on the tensor cores (0: the CUDA-core kernel, for comparisons)
window_attention_tc = os.environ.get("TLLM_WINDOW_ATTENTION_TC", "1") != "0"
# ... and its key tiles in several runs per row tile when the grid would not fill the SMs (decoded tokens); 0: one run
window_attention_splits = os.environ.get("TLLM_WINDOW_ATTENTION_SPLITS", "1") != "0"


def _keep(struct):
    """A by-reference argument that stays valid for as long as a tape of launches holds it."""
    ref = ctypes.byref(struct)
    return ref


def window_pool_attention(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                          k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                          pool_k: Optional[torch.Tensor], pool_v: Optional[torch.Tensor],
                          pool_table: Optional[torch.Tensor], batch, out: torch.Tensor, scale: float,
                          softcap: Optional[float], head_bias: torch.Tensor, window: Optional[int], pool: Optional[int],
                          freq_v: Optional[torch.Tensor], workspace=None) -> None:
    """Attention without softmax: out[t, h] = sum over visible keys of sigmoid(cap(q . k * scale) + head_bias[h]) * v,
    cap(s) = softcap * tanh(s / softcap) (None: s).  Visible to position i: tokens j with 0 <= i - j < window (None:
    all j <= i) and, with `pool`, the block rows b of pool_k / pool_v with b * pool + pool - 1 <= i - window.  With
    `freq_v` the head's output is turned back by the query's position (value m with m + value_dim / 2, angle
    -i * freq_v[m]).  The queries are the first num_heads * key_dim values of every row of `qkv`."""
    _need_cuda(qkv, k_cache, v_cache, block_table, pool_k, pool_v, pool_table, out, head_bias, freq_v)
    _i32(block_table, "block_table")
    _i32(pool_table, "pool_table")
    t = qkv.shape[0]
    _paged("window_pool_attention", k_cache, num_kv_heads, key_dim)
    _paged("window_pool_attention", v_cache, num_kv_heads, value_dim)
    if qkv.stride(1) != 1 or qkv.shape[1] < num_heads * key_dim or out.shape != (t, num_heads * value_dim) or \
            not out.is_contiguous() or out.dtype != qkv.dtype or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or \
            head_bias.dtype != torch.float32 or head_bias.numel() != num_heads or \
            (freq_v is not None and (freq_v.dtype != torch.float32 or freq_v.numel() * 2 != value_dim)):
        raise KernelError("window_pool_attention: shapes or dtypes do not fit")
    a = _WinArgs()
    a.qkv, a.row_stride, a.nh, a.nkv, a.kd, a.vd = qkv.data_ptr(), qkv.stride(0), num_heads, num_kv_heads, key_dim, value_dim
    a.k, a.v, a.table, a.max_blocks = k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1]
    a.k_page_stride, a.k_head_stride = k_cache.stride(0), k_cache.stride(1)
    a.v_page_stride, a.v_head_stride = v_cache.stride(0), v_cache.stride(1)
    if pool:
        if pool_k is None or pool_v is None or pool_table is None or window is None:
            raise KernelError("window_pool_attention: pooled blocks need their cache, their table and a window")
        _paged("window_pool_attention", pool_k, num_kv_heads, key_dim)
        _paged("window_pool_attention", pool_v, num_kv_heads, value_dim)
        if pool_k.dtype != qkv.dtype or pool_v.dtype != qkv.dtype or pool_k.shape[2] != k_cache.shape[2]:
            raise KernelError("window_pool_attention: the block cache differs in dtype or page size")
        a.pk, a.pv, a.ptable, a.pmax_blocks = pool_k.data_ptr(), pool_v.data_ptr(), pool_table.data_ptr(), pool_table.shape[1]
        a.pk_page_stride, a.pk_head_stride = pool_k.stride(0), pool_k.stride(1)
        a.pv_page_stride, a.pv_head_stride = pool_v.stride(0), pool_v.stride(1)
    a.page_size = k_cache.shape[2]
    a.positions, a.token_request, a.out = batch.positions.data_ptr(), batch.token_request.data_ptr(), out.data_ptr()
    a.scale, a.cap, a.head_bias = scale, (softcap or 0.0), head_bias.data_ptr()
    a.window, a.pool, a.fv, a.n_tokens = (window or 0), (pool or 0), (None if freq_v is None else freq_v.data_ptr()), t
    heads_per_kv = num_heads // num_kv_heads
    if qkv.dtype == torch.bfloat16 and window_attention_tc and not force_generic and key_dim % 16 == 0 and \
            value_dim % 16 == 0 and key_dim <= 128 and value_dim <= 128 and heads_per_kv <= 64 and qkv.stride(0) % 8 == 0 and \
            qkv.data_ptr() % 16 == 0 and getattr(batch, "cu_q", None) is not None:
        # bfloat16: the tensor-core kernel compiled for this pair of sizes (prompt portions and decoded tokens alike)
        lib = build.load_library("window_attention_mma", flags=(f"-DTLLM_HEAD_DIM={key_dim}", f"-DTLLM_VALUE_DIM={value_dim}"))
        # few CTAs and many keys (decoded tokens): the key tiles of a row tile in runs that add into a 32-bit buffer
        splits, acc = 1, None
        max_kv = getattr(batch, "max_kv_len", 0)
        if workspace is not None and window_attention_splits and max_kv:
            tokens_per_tile = 64 // heads_per_kv
            ctas = -(-batch.max_q_len // tokens_per_tile) * num_kv_heads * batch.num_requests
            keys = (min(max_kv, window) if window else max_kv) + (max_kv // pool if pool else 0)
            tiles = -(-keys // 32)
            splits = max(1, min(16, sm_count(qkv.device) // ctas, tiles // 4))
            if splits > 1:
                acc = workspace.get_zeroed("window_attn_acc", (t, num_heads * value_dim))
        _call(lib, lib.tllm_window_pool_attention_mma, _keep(a), _ptr(batch.cu_q), _ptr(batch.q_start), batch.num_requests,
              batch.max_q_len, splits, _ptr(acc), _stream())
        return
    lib = build.load_library("window_attention")
    _call(lib, lib.tllm_window_pool_attention, _keep(a), _code(qkv.dtype), _stream())


def gelu(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = 0.5 x (1 + erf(x / sqrt 2)) element by element (`out` may be `x`)."""
    _need_cuda(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("gelu: shapes or dtypes do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_gelu, _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _code(x.dtype), _stream())


def moe_route(logits: torch.Tensor, num_experts: int, correction: Optional[torch.Tensor], scale: float, ids: torch.Tensor,
              weights: torch.Tensor, softmax: bool = False) -> None:
    """Per token: s = sigmoid(logits[t, :num_experts]), or softmax over the experts with softmax=True; ids[t] = the `top`
    experts with the largest s + correction (None: s; ties: the lower index), weights[t] = their s * scale.  logits
    float32 (further columns are ignored), ids int32 [T, top], weights float32 [T, top]."""
    _need_cuda(logits, correction, ids, weights)
    t, top = ids.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or logits.shape[0] != t or logits.shape[1] < num_experts or \
            (correction is not None and (correction.dtype != torch.float32 or correction.numel() != num_experts)) or \
            ids.dtype != torch.int32 or \
            weights.dtype != torch.float32 or weights.shape != ids.shape or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("moe_route: shapes or dtypes do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_moe_route, _ptr(logits), logits.stride(0), num_experts, _ptr(correction), ctypes.c_float(scale), top,
          _ptr(ids), _ptr(weights), t, 1 if softmax else 0, _stream())


def moe_tile_rows(pairs: int, num_experts: int, tensor_cores: bool = False) -> int:
    """Rows per tile of the grouped product: 16 while an expert gets few rows (decode), else 64; 128 where the
    tensor-core kernel runs and an expert gets some hundred rows."""
    if pairs <= 16 * num_experts:
        return 16
    return 128 if tensor_cores and moe_mma and not force_generic and moe_wide_tiles and pairs >= 192 * num_experts else 64


def moe_max_tiles(pairs: int, num_experts: int, tile: int) -> int:
    """The most tiles `pairs` rows can fill when grouped by expert: every expert may end in one partial tile."""
    return pairs // tile + min(num_experts, pairs)


def moe_align(ids: torch.Tensor, num_experts: int, tile: int, sorted_rows: torch.Tensor, tile_expert: torch.Tensor,
              pair_pos: Optional[torch.Tensor] = None) -> None:
    """Groups the pairs (token, choice), numbered in the order of `ids`, by expert into tiles of `tile` rows:
    sorted_rows[tiles * tile] (pair numbers, -1 = padding) and tile_expert[tiles] (-1 = no such tile); with `pair_pos`
    (int32 [pairs]) also where every pair's row lies in that order."""
    _need_cuda(ids, sorted_rows, tile_expert, pair_pos)
    _i32(pair_pos, "pair_pos")
    if pair_pos is not None and pair_pos.numel() != ids.numel():
        raise KernelError("moe_align: pair_pos does not fit")
    _i32(ids, "ids")
    _i32(sorted_rows, "sorted_rows")
    _i32(tile_expert, "tile_expert")
    tiles = tile_expert.numel()
    if sorted_rows.numel() != tiles * tile or tiles < moe_max_tiles(ids.numel(), num_experts, tile):
        raise KernelError("moe_align: the tile buffers do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_moe_align, _ptr(ids), ids.numel(), num_experts, tile, tiles, _ptr(sorted_rows), _ptr(tile_expert),
          _ptr(pair_pos), _stream())


# Grouped products of prompt portions on tcgen05: at least this many (token, choice) pairs per expert on average
# (tiles are 128 rows there, so fewer rows would mostly be padding); 0: never
moe_tc_rows_per_expert = int(os.environ.get("TLLM_MOE_TC_ROWS", "32"))
MOE_TC_TILE = 128


def moe_tc_preferred(pairs: int, num_experts: int, dtype: torch.dtype, *sizes: int) -> bool:
    """Whether a step's grouped products run on the tcgen05 kernel: bfloat16, enough rows per expert, sizes TMA takes."""
    return (dtype == torch.bfloat16 and not force_generic and moe_tc_rows_per_expert > 0 and
            pairs >= moe_tc_rows_per_expert * num_experts and all(x % 8 == 0 for x in sizes))


def moe_gather(a: torch.Tensor, sorted_rows: torch.Tensor, tile_expert: torch.Tensor, tile: int, out: torch.Tensor,
               rows_per_input: int = 1) -> None:
    """out[p] = a[sorted_rows[p] // rows_per_input] (zeros where sorted_rows is -1; tiles that do not exist are left
    alone): the grouped order's input rows made contiguous.  bfloat16, rows of a multiple of 8 values."""
    _need_cuda(a, sorted_rows, tile_expert, out)
    k = a.shape[1]
    if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or a.stride(1) != 1 or not out.is_contiguous() or \
            out.shape != (sorted_rows.numel(), k) or sorted_rows.numel() != tile_expert.numel() * tile:
        raise KernelError("moe_gather: shapes or dtypes do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_moe_gather, _ptr(a), a.stride(0), _ptr(sorted_rows), _ptr(tile_expert), tile, tile_expert.numel(),
          rows_per_input, _ptr(out), k, _stream())


def moe_linear_tc(a: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, out: torch.Tensor, gelu: bool = False) -> None:
    """The grouped product on tcgen05: a [tiles * 128, K] bfloat16 in the grouped order (every tile of 128 rows one
    expert's), w [experts, N, K]; out [tiles * 128, N]: bfloat16 of GELU(sums) with gelu=True, else float32 sums."""
    _need_cuda(a, w, tile_expert, out)
    _i32(tile_expert, "tile_expert")
    experts, n, k = w.shape
    rows = tile_expert.numel() * MOE_TC_TILE
    if a.shape != (rows, k) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or \
            a.stride(1) != 1 or out.shape != (rows, n) or out.stride(1) != 1 or \
            out.dtype != (torch.bfloat16 if gelu else torch.float32):
        raise KernelError("moe_linear_tc: shapes or dtypes do not fit")
    lib = build.load_library("linear_tc")
    _call(lib, lib.tllm_linear_tc_grouped, _ptr(a), _ptr(w), _ptr(out), rows, n, k, a.stride(0), out.stride(0), experts,
          _ptr(tile_expert), 10 if gelu else EPI_F32, _ptr(status_word(a.device)), _stream())


# bfloat16 grouped products on the tensor cores (0: the FFMA kernel, for comparisons)
moe_mma = os.environ.get("TLLM_MOE_MMA", "1") != "0"
# tiles of 128 rows where an expert gets some hundred rows: measured no faster than tiles of 64 (240 against 225 us for
# 8,192 rows of 2,048 x 1,408) and they pad more, so they are off unless asked for
moe_wide_tiles = os.environ.get("TLLM_MOE_TILE_128", "0") == "1"


def moe_linear(a: torch.Tensor, w: torch.Tensor, sorted_rows: torch.Tensor, tile_expert: torch.Tensor, tile: int,
               out: torch.Tensor, rows_per_input: int = 1, gelu: bool = False) -> None:
    """out[p] = act(w[expert of p] . a[p // rows_per_input]) for every pair p named in sorted_rows; w [experts, N, K],
    out [pairs, N] in a's dtype or float32; act is the exact GELU or nothing."""
    _need_cuda(a, w, sorted_rows, tile_expert, out)
    n, k = w.shape[1], w.shape[2]
    if a.shape[1] != k or a.stride(1) != 1 or a.dtype != w.dtype or not w.is_contiguous() or out.shape[1] != n or \
            not out.is_contiguous() or out.dtype not in (a.dtype, torch.float32):
        raise KernelError("moe_linear: shapes or dtypes do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_moe_linear, _ptr(a), a.stride(0), _ptr(w), _ptr(sorted_rows), _ptr(tile_expert), _ptr(out), n, k,
          rows_per_input, tile, tile_expert.numel(), 1 if gelu else 0, _code(a.dtype), _code(out.dtype),
          1 if (moe_mma and not force_generic) else 0, _stream())


def moe_combine(y: torch.Tensor, weights: torch.Tensor, shared: Optional[torch.Tensor], logits: Optional[torch.Tensor],
                gate_col: int, resid: torch.Tensor, pair_pos: Optional[torch.Tensor] = None) -> None:
    """resid[t] += sum_c weights[t, c] * y[t * top + c] + sigmoid(logits[t, gate_col]) * shared[t] (the last term only
    with `shared`); all float32.  With `pair_pos` (int32 [T * top]) y is in the grouped order: pair p lies in row pair_pos[p]."""
    _need_cuda(y, weights, shared, logits, resid, pair_pos)
    _i32(pair_pos, "pair_pos")
    t, width = resid.shape
    top = weights.shape[1]
    if (pair_pos is None and y.shape != (t * top, width)) or y.shape[1] != width or \
            (pair_pos is not None and pair_pos.numel() != t * top) or any(x.dtype != torch.float32 or not x.is_contiguous() for x in (y, weights, resid)) or \
            (shared is not None and (shared.shape != resid.shape or shared.dtype != torch.float32 or not shared.is_contiguous()
                                     or logits is None or logits.dtype != torch.float32 or logits.shape[1] <= gate_col)):
        raise KernelError("moe_combine: shapes or dtypes do not fit")
    lib = build.load_library("moe")
    _call(lib, lib.tllm_moe_combine, _ptr(y), _ptr(weights), top, _ptr(shared), _ptr(logits),
          0 if logits is None else logits.stride(0), gate_col, _ptr(resid), t, width, _ptr(pair_pos), _stream())


# ----------------------------------------------------------------------------- attention without rotate-half, delta rule


def qk_norm_kv_write(proj: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int, key_dim: int,
                     value_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                     bias_q: Optional[torch.Tensor] = None, bias_k: Optional[torch.Tensor] = None,
                     bias_v: Optional[torch.Tensor] = None, norm_q: Optional[torch.Tensor] = None,
                     norm_k: Optional[torch.Tensor] = None, eps: float = 0.0, stretch_coef: float = 0.0,
                     stretch_every: int = 0, freq: Optional[torch.Tensor] = None, rot_pairs: bool = False,
                     rot_mag: float = 1.0) -> None:
    """Rows of `proj` begin with num_heads query heads and num_kv_heads key heads of key_dim values, then num_kv_heads
    value heads of value_dim values.  Biases (float32) are added; with norm weights (float32 [key_dim], shared by the
    heads) query and key heads become x / sqrt(mean(x^2) + eps) * weight; with stretch_every > 0 the query at position
    p is multiplied by 1 + stretch_coef * ln(floor((p + 1) / stretch_every) + 1).  With `freq` (float32, n values) the
    first 2n values of every query and key head are then turned by positions[t] * freq[i] in 32-bit, value i with
    i + n (rot_pairs: value 2i with 2i + 1), cos and sin multiplied by rot_mag.  Queries are rewritten in place, keys
    and values go to their pages."""
    _need_cuda(proj, positions, k_cache, v_cache, slot_mapping, bias_q, bias_k, bias_v, norm_q, norm_k, freq)
    if freq is not None and (freq.dtype != torch.float32 or not freq.is_contiguous() or 2 * freq.numel() > key_dim):
        raise KernelError("qk_norm_kv_write: the frequencies are contiguous float32, at most half a head's size of them")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t = proj.shape[0]
    if proj.stride(1) != 1 or proj.shape[1] < (num_heads + num_kv_heads) * key_dim + num_kv_heads * value_dim:
        raise KernelError("qk_norm_kv_write: the rows of the projection do not fit")
    _paged("qk_norm_kv_write", k_cache, num_kv_heads, key_dim)
    _paged("qk_norm_kv_write", v_cache, num_kv_heads, value_dim)
    if k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype or k_cache.shape[2] != v_cache.shape[2]:
        raise KernelError("qk_norm_kv_write: cache dtype or page size does not fit")
    for name, b, n in (("query bias", bias_q, num_heads * key_dim), ("key bias", bias_k, num_kv_heads * key_dim),
                       ("value bias", bias_v, num_kv_heads * value_dim), ("query norm", norm_q, key_dim),
                       ("key norm", norm_k, key_dim)):
        if b is not None and (b.dtype != torch.float32 or b.numel() != n or not b.is_contiguous()):
            raise KernelError(f"qk_norm_kv_write: the {name} must be {n} contiguous float32 values")
    ll = ctypes.c_longlong
    lib = build.load_library("attention_prep")
    _call(lib, lib.tllm_qk_norm_kv_write, _ptr(proj), proj.stride(0), num_heads, num_kv_heads, key_dim, value_dim,
          _ptr(bias_q), _ptr(bias_k), _ptr(bias_v), _ptr(norm_q), _ptr(norm_k), ctypes.c_float(eps),
          ctypes.c_float(stretch_coef), int(stretch_every), _ptr(positions), _ptr(k_cache), _ptr(v_cache),
          _ptr(slot_mapping), k_cache.shape[2], ll(k_cache.stride(0)), ll(k_cache.stride(1)), ll(v_cache.stride(0)),
          ll(v_cache.stride(1)), t, _ptr(freq), 0 if freq is None else 2 * freq.numel(), 1 if rot_pairs else 0,
          ctypes.c_float(rot_mag), _code(proj.dtype), _stream())


def latent_kv_write(proj: torch.Tensor, positions: torch.Tensor, num_heads: int, plain_dim: int, rot_part: int,
                    rank: int, rot_dims: int, freq: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float,
                    q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                    slot_mapping: Optional[torch.Tensor], rot_mag: float = 1.0) -> None:
    """Rows of `proj`: num_heads query heads of [plain_dim | rot_part] values, then `rank` latent values and rot_part
    key values shared by the heads.  The latent, normed with `norm_weight`, becomes the first `rank` values of the
    token's key row and its whole value row; the key's part and every query head's part are rotated pairwise (value
    2i with 2i + 1, i < rot_dims / 2) by positions[t] * freq[i]; the key part is written behind the latent, the query
    parts to q_out[t, head, rank:] (q_out [T, num_heads, rank + rot_part]).  cos and sin are multiplied by rot_mag.
    Without caches (k_cache None) the rows hold the query heads only and only their parts are turned: the form of a
    mixer that reads what another layer cached."""
    _need_cuda(proj, positions, freq, norm_weight, q_out, k_cache, v_cache, slot_mapping)
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t = proj.shape[0]
    kd = rank + rot_part
    if k_cache is None:
        if proj.stride(1) != 1 or proj.shape[1] < num_heads * (plain_dim + rot_part) or q_out.shape != (t, num_heads, kd) or \
                not q_out.is_contiguous() or q_out.dtype != proj.dtype or \
                (rot_dims and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != rot_dims)):
            raise KernelError("latent_kv_write: the rows of the projection or of the query buffer do not fit")
        lib = build.load_library("attention_prep")
        _call(lib, lib.tllm_latent_kv_write, _ptr(proj), proj.stride(0), num_heads, plain_dim, rot_part, rank, rot_dims,
              _ptr(None), _ptr(freq if rot_dims else None), ctypes.c_float(eps), _ptr(positions), _ptr(q_out),
              _ptr(None), _ptr(None), _ptr(None), 1, ctypes.c_longlong(0), ctypes.c_longlong(0), t,
              ctypes.c_float(rot_mag), _code(proj.dtype), _stream())
        return
    if proj.stride(1) != 1 or proj.shape[1] < num_heads * (plain_dim + rot_part) + kd or \
            q_out.shape != (t, num_heads, kd) or not q_out.is_contiguous() or q_out.dtype != proj.dtype:
        raise KernelError("latent_kv_write: the rows of the projection or of the query buffer do not fit")
    _paged("latent_kv_write", k_cache, 1, kd)
    _paged("latent_kv_write", v_cache, 1, rank)
    if k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype or k_cache.shape[2] != v_cache.shape[2] or \
            norm_weight.dtype != torch.float32 or norm_weight.numel() != rank or \
            (rot_dims and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != rot_dims)):
        raise KernelError("latent_kv_write: cache, norm weight or frequency table does not fit")
    ll = ctypes.c_longlong
    lib = build.load_library("attention_prep")
    _call(lib, lib.tllm_latent_kv_write, _ptr(proj), proj.stride(0), num_heads, plain_dim, rot_part, rank, rot_dims,
          _ptr(norm_weight), _ptr(freq if rot_dims else None), ctypes.c_float(eps), _ptr(positions), _ptr(q_out),
          _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), k_cache.shape[2], ll(k_cache.stride(0)), ll(v_cache.stride(0)),
          t, ctypes.c_float(rot_mag), _code(proj.dtype), _stream())


def head_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """One small product per head in one launch: out[t, h, :] = w[h] . a[t, h, :].  a [T, heads, K] and out
    [T, heads, N] are views whose last dimension is contiguous (rows of tokens with the heads side by side, at any
    row stride and any distance between heads); w [heads, N, K] contiguous, of a's dtype; out of a's dtype or float32.
    bfloat16 with even K and even offsets runs on mma.sync tiles read straight from global memory, everything else
    on FFMA tiles; either way an output's sum runs over ascending k whatever else is in the batch."""
    _need_cuda(a, w, out)
    t, heads, k = a.shape
    n = w.shape[1]
    if w.shape != (heads, n, k) or not w.is_contiguous() or w.dtype != a.dtype or out.shape != (t, heads, n) or \
            a.stride(2) != 1 or out.stride(2) != 1 or out.dtype not in (a.dtype, torch.float32):
        raise KernelError("head_linear: shapes or dtypes do not fit")
    lib = build.load_library("head_linear")
    ll = ctypes.c_longlong
    _call(lib, lib.tllm_head_linear, _ptr(a), ll(a.stride(0)), a.stride(1), _ptr(w), _ptr(out), ll(out.stride(0)),
          out.stride(1), t, heads, n, k, _code(a.dtype), _code(out.dtype), 0 if force_generic else 1, _stream())


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, value_dim: int, out: torch.Tensor) -> None:
    """out[t, h, :] = x[t, h, :] * sigmoid(gate[t, ...]): `gate` [T, heads * value_dim] gates every value, `gate`
    [T, heads] every head as a whole.  x float32, gate (a row slice is fine) and out in the engine's dtype."""
    _need_cuda(x, gate, out)
    t = x.shape[0]
    per_head = gate.shape[1] == heads and value_dim != 1
    if x.dtype != torch.float32 or not x.is_contiguous() or x.shape != (t, heads * value_dim) or out.shape != x.shape or \
            not out.is_contiguous() or out.dtype != gate.dtype or gate.stride(1) != 1 or gate.shape[0] != t or \
            gate.shape[1] not in (heads, heads * value_dim):
        raise KernelError("sigmoid_gate: shapes or dtypes do not fit")
    lib = build.load_library("attention_prep")
    _call(lib, lib.tllm_sigmoid_gate, _ptr(x), _ptr(gate), gate.stride(0), 1 if per_head else 0, _ptr(out),
          ctypes.c_longlong(t), heads, value_dim, _code(out.dtype), _stream())


PREPARE_MODES = {"delta": 0, "state_space": 1, "channel_decay": 2}


def delta_prepare(proj: torch.Tensor, taps: torch.Tensor, kept: torch.Tensor, batch, heads: int, kv_heads: int,
                  key_dim: int, value_dim: int, beta_col: int, a_col: int, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  q_scale: float, unit_eps: float, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gb: torch.Tensor,
                  mode: str = "delta", conv_bias: Optional[torch.Tensor] = None, decay_in: Optional[torch.Tensor] = None,
                  gk: Optional[torch.Tensor] = None) -> None:
    """The inputs of the delta rule from the fused projection.  The first kv_heads * key_dim * 2 + heads * value_dim
    columns of `proj` are the channels [queries | keys | values]; each is filtered over time with its row of `taps`
    (float32 [channels, n]; the last column meets the current token; ahead of the step's tokens stand the inputs in
    kept[slot] (float32 [slots, n - 1, channels], oldest first)), then SiLU.  Query and key heads are divided by
    sqrt(sum(x^2) + unit_eps), queries also multiplied by q_scale.  Columns beta_col + h and a_col + h hold the step
    size's and the decay's inputs: gb[t, h] = (exp(-exp(a_log[h]) softplus(a + dt_bias[h])), sigmoid(b)).  q, k, v, gb
    are float32.
    mode "channel_decay": the decay is one per head and key channel, gk[t, h, c] = exp(-exp(a_log[h]) softplus(decay_in[t, h, c]
    + dt_bias[h, c])) from float32 rows `decay_in`, and gb[t, h] = (1, sigmoid(b)); a_col is not read.
    mode "state_space": the channels are [values | keys | queries], the filters add `conv_bias` (float32 [channels]),
    nothing is made a unit vector, and gb[t, h] = (exp(-exp(a_log[h]) dt), dt) with dt = softplus(b + dt_bias[h])."""
    _need_cuda(proj, taps, kept, a_log, dt_bias, q, k, v, gb, conv_bias, decay_in, gk)
    t = proj.shape[0]
    channels = 2 * kv_heads * key_dim + heads * value_dim
    n = taps.shape[1]
    if mode not in PREPARE_MODES:
        raise KernelError(f"delta_prepare: unknown mode {mode!r} (known: {', '.join(PREPARE_MODES)})")
    qk = kv_heads * key_dim
    q_c0, k_c0, v_c0 = (heads * value_dim + qk, heads * value_dim, 0) if mode == "state_space" else (0, qk, 2 * qk)
    n_bias = heads * key_dim if mode == "channel_decay" else heads
    if (mode == "channel_decay") != (decay_in is not None and gk is not None) or \
            (conv_bias is not None and (conv_bias.dtype != torch.float32 or conv_bias.numel() != channels or not conv_bias.is_contiguous())) or \
            any(x is not None and (x.dtype != torch.float32 or not x.is_contiguous() or x.shape != (t, heads * key_dim)) for x in (decay_in, gk)):
        raise KernelError("delta_prepare: the decays' rows or the filters' bias do not fit the mode")
    if proj.stride(1) != 1 or proj.shape[1] < max(channels, beta_col + heads, a_col + heads) or \
            taps.dtype != torch.float32 or taps.shape != (channels, n) or not taps.is_contiguous() or \
            kept.dtype != torch.float32 or not kept.is_contiguous() or tuple(kept.shape[1:]) != (max(n - 1, 1), channels) or \
            any(x.dtype != torch.float32 or not x.is_contiguous() for x in (a_log, dt_bias, q, k, v, gb)) or \
            a_log.numel() != heads or dt_bias.numel() != n_bias or q.shape != (t, kv_heads * key_dim) or k.shape != q.shape or \
            v.shape != (t, heads * value_dim) or gb.shape != (t, heads, 2):
        raise KernelError("delta_prepare: shapes or dtypes do not fit")
    lib = build.load_library("delta_rule")
    _call(lib, lib.tllm_delta_prepare, _ptr(proj), proj.stride(0), _ptr(taps), n, _ptr(kept), _ptr(batch.slots),
          _ptr(batch.cu_q), _ptr(batch.token_request), heads, kv_heads, key_dim, value_dim, beta_col, a_col, _ptr(a_log),
          _ptr(dt_bias), ctypes.c_float(q_scale), ctypes.c_float(unit_eps), _ptr(q), _ptr(k), _ptr(v), _ptr(gb), t,
          q_c0, k_c0, v_c0, _ptr(conv_bias), 0 if mode == "state_space" else 1, PREPARE_MODES[mode], _ptr(decay_in), _ptr(gk),
          _code(proj.dtype), _stream())


def conv_state_update(proj: torch.Tensor, kept: torch.Tensor, batch, n_taps: int, channels: int) -> None:
    """kept[slot] <- the last n_taps - 1 inputs of every channel after the step's tokens (what was kept before moves
    up when the step brought fewer tokens than that)."""
    _need_cuda(proj, kept)
    if proj.stride(1) != 1 or proj.shape[1] < channels or kept.dtype != torch.float32 or not kept.is_contiguous() or \
            tuple(kept.shape[1:]) != (max(n_taps - 1, 1), channels):
        raise KernelError("conv_state_update: shapes or dtypes do not fit")
    lib = build.load_library("delta_rule")
    _call(lib, lib.tllm_conv_state_update, _ptr(proj), proj.stride(0), _ptr(kept), _ptr(batch.slots), _ptr(batch.cu_q),
          n_taps, channels, batch.num_requests, _code(proj.dtype), _stream())


def delta_rule_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gb: torch.Tensor, state: torch.Tensor, batch,
                    heads: int, kv_heads: int, key_dim: int, value_dim: int, out: torch.Tensor, mode: str = "delta",
                    gk: Optional[torch.Tensor] = None) -> None:
    """Per head and token, in order: S <- g S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q, with (g, beta) =
    gb[t, h]; head h reads query/key head h // (heads / kv_heads).  All float32; state [slots, heads, value_dim,
    key_dim] (the transpose of S) is carried from step to step.  mode "channel_decay": S <- diag(gk[t, h]) S instead of
    g S (gk float32 [T, heads * key_dim]).  mode "state_space": no correction, u = beta v."""
    _need_cuda(q, k, v, gb, state, out, gk)
    if mode not in PREPARE_MODES or (mode == "channel_decay") != (gk is not None) or \
            (gk is not None and (gk.dtype != torch.float32 or not gk.is_contiguous() or gk.shape != (q.shape[0], heads * key_dim))):
        raise KernelError(f"delta_rule_scan: mode {mode!r} and the decays per key channel do not fit")
    t = q.shape[0]
    if any(x.dtype != torch.float32 or not x.is_contiguous() for x in (q, k, v, gb, state, out)) or \
            q.shape != (t, kv_heads * key_dim) or k.shape != q.shape or v.shape != (t, heads * value_dim) or \
            gb.shape != (t, heads, 2) or out.shape != v.shape or tuple(state.shape[1:]) != (heads, value_dim, key_dim):
        raise KernelError("delta_rule_scan: shapes or dtypes do not fit")
    lib = build.load_library("delta_rule")
    _call(lib, lib.tllm_delta_rule_scan, _ptr(q), _ptr(k), _ptr(v), _ptr(gb), _ptr(state), _ptr(batch.slots),
          _ptr(batch.cu_q), _ptr(out), heads, kv_heads, key_dim, value_dim, batch.num_requests, PREPARE_MODES[mode],
          _ptr(gk), _stream())


def bigram_add(tokens: torch.Tensor, table: torch.Tensor, last: torch.Tensor, batch, out: torch.Tensor, mul_prev: int,
               mul_cur: int) -> None:
    """out[t] += table[(prev_t * mul_prev + tokens[t] * mul_cur) mod buckets] with buckets = rows of `table` - 1 and
    prev_t the token before t in its sequence; a sequence's first token takes the table's last row.  The token before
    a step's first one is last[slot] (int32 [slots, 1]), which this launch also replaces by the step's last token."""
    _need_cuda(tokens, table, last, out)
    _i32(tokens, "tokens")
    _i32(last, "last")
    t, h = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous() or table.shape[1] != h or \
            table.shape[0] < 2 or tokens.numel() != t or last.numel() != last.shape[0]:
        raise KernelError("bigram_add: shapes or dtypes do not fit")
    ll = ctypes.c_longlong
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_bigram_add, _ptr(tokens), _ptr(batch.token_request), _ptr(batch.cu_q), _ptr(batch.q_start),
          _ptr(batch.slots), _ptr(last), _ptr(table), _ptr(out), t, h, ll(table.shape[0] - 1), ll(mul_prev), ll(mul_cur),
          _code(table.dtype), _stream())


UNARY_ACTS = {"copy": 0, "relu2": 1}


def unary(x: torch.Tensor, out: torch.Tensor, act: str = "copy") -> None:
    """out = act(x) element by element, computed in 32-bit and rounded once to out's dtype: "copy" (x in another
    dtype) or "relu2" (relu(x)^2).  x float32 or of out's dtype."""
    _need_cuda(x, out)
    if x.shape != out.shape or not x.is_contiguous() or not out.is_contiguous() or act not in UNARY_ACTS or \
            x.dtype not in (torch.float32, out.dtype):
        raise KernelError("unary: shapes, dtypes or activation do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_unary, _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _code(x.dtype), _code(out.dtype),
          UNARY_ACTS[act], _stream())


def scaled_add(x: torch.Tensor, scale: float, resid: torch.Tensor, clear: bool = True) -> None:
    """resid += scale * x, all float32; clear=True hands `x` back zeroed (a branch buffer that products add into)."""
    _need_cuda(x, resid)
    if x.dtype != torch.float32 or resid.dtype != torch.float32 or x.shape != resid.shape or not x.is_contiguous() or \
            not resid.is_contiguous():
        raise KernelError("scaled_add: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_scaled_add, _ptr(x), _ptr(resid), ctypes.c_longlong(x.numel()), ctypes.c_float(scale),
          1 if clear else 0, _stream())


def gated_group_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, parts: int, value_dim: int, eps: float,
                     out: torch.Tensor, skip_x: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None) -> None:
    """y = (o + skip[h] * skip_x) * silu(gate), then each of `parts` equal parts of a row is divided by its root mean
    square (eps inside the root) and multiplied by `weight`; the gate comes before the norm.  o, skip_x float32
    [T, width], skip float32 [width / value_dim] (one per head), gate (a row slice is fine) and out [T, width] in the
    engine's dtype, weight float32 [width]."""
    _need_cuda(o, gate, weight, out, skip_x, skip)
    t, width = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or gate.shape != o.shape or gate.stride(1) != 1 or \
            out.shape != o.shape or not out.is_contiguous() or out.dtype != gate.dtype or weight.dtype != torch.float32 or \
            weight.numel() != width or width % parts or width % value_dim or (skip_x is None) != (skip is None) or \
            (skip_x is not None and (skip_x.dtype != torch.float32 or skip_x.shape != o.shape or not skip_x.is_contiguous() or
                                     skip.dtype != torch.float32 or skip.numel() != width // value_dim)):
        raise KernelError("gated_group_norm: shapes or dtypes do not fit")
    lib = build.load_library("delta_rule")
    _call(lib, lib.tllm_gated_group_norm, _ptr(o), _ptr(skip_x), _ptr(skip), _ptr(gate), gate.stride(0), _ptr(weight),
          _ptr(out), ctypes.c_longlong(t), width, parts, value_dim, ctypes.c_float(eps), _code(out.dtype), _stream())


# The mixed-scores attention on the tensor cores for bfloat16 (0: always the CUDA-core kernel), and the most runs a
# decode step's key tiles are cut into (0 or 1: one run)
attention_talk_tc = os.environ.get("TLLM_ATTENTION_TALK_TC", "1") != "0"
attention_talk_splits = int(os.environ.get("TLLM_ATTENTION_TALK_SPLITS", "16"))
attention_talk_stages = int(os.environ.get("TLLM_ATTENTION_TALK_STAGES", "2"))   # staged key tiles of the tensor-core kernel (1 or 2)


def attention_talk(q: torch.Tensor, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, block_table: torch.Tensor, batch, mix: torch.Tensor, out: torch.Tensor,
                   window: Optional[int] = None, sink: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None, mix_log2: Optional[torch.Tensor] = None, workspace=None) -> None:
    """Attention whose heads' scores are mixed before the softmax: z_h = sum_g mix[h, g] (q_g . k), softmax over the
    visible keys (the last `window`, or all earlier ones), optionally with exp(sink[h]) in the denominator, head h's
    output optionally times sigmoid(gate[t, h]).  q: rows that begin with the query heads; caches [pages,
    num_kv_heads, page_size, key_dim | value_dim]; mix float32 [heads, heads] (the score scale folded in); out
    [T, heads * value_dim] in the cache's dtype or float32.  Everything but the reads is 32-bit.
    bfloat16 with `mix_log2` (mix times log2(e), made once by the caller), at most 16 heads and sizes that are multiples
    of 16 up to 256 runs on the tensor cores (products of bfloat16 queries, keys, values and two-part weights; sums,
    mixing and softmax in 32-bit); `workspace` (the step's named buffers) lets a step of decoded tokens cut the keys
    into runs that separate CTAs walk (needs batch.max_kv_len, an upper bound of the contexts).  Everything else runs
    on the CUDA cores in 32-bit, where the result does not depend on how a prompt was cut."""
    _need_cuda(q, k_cache, v_cache, block_table, mix, out, sink, gate)
    _i32(block_table, "block_table")
    t = q.shape[0]
    _paged("attention_talk", k_cache, num_kv_heads, key_dim)
    _paged("attention_talk", v_cache, num_kv_heads, value_dim)
    if q.stride(1) != 1 or q.shape[1] < num_heads * key_dim or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or \
            k_cache.shape[2] != v_cache.shape[2] or mix.dtype != torch.float32 or mix.shape != (num_heads, num_heads) or \
            not mix.is_contiguous() or out.shape != (t, num_heads * value_dim) or not out.is_contiguous() or \
            out.dtype not in (q.dtype, torch.float32) or \
            (sink is not None and (sink.dtype != torch.float32 or sink.numel() != num_heads or not sink.is_contiguous())) or \
            (gate is not None and (gate.dtype != q.dtype or gate.shape != (t, num_heads) or gate.stride(1) != 1)):
        raise KernelError("attention_talk: shapes or dtypes do not fit")
    ll = ctypes.c_longlong
    if q.dtype == torch.bfloat16 and mix_log2 is not None and attention_talk_tc and not force_generic and num_heads <= 16 and \
            key_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= key_dim <= 256 and 16 <= value_dim <= 256 and \
            q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0:
        lib = build.load_library("attention_talk_mma", flags=(f"-DTLLM_HEAD_DIM={key_dim}", f"-DTLLM_VALUE_DIM={value_dim}"))
        lib.tllm_attention_talk_mma_smem.restype = ctypes.c_longlong
        if lib.tllm_attention_talk_mma_smem(num_heads, num_kv_heads, 1) <= 220 * 1024:
            if mix_log2.dtype != torch.float32 or mix_log2.shape != mix.shape or not mix_log2.is_contiguous():
                raise KernelError("attention_talk: mix_log2 does not fit mix")
            splits, part = 1, None
            if workspace is not None and batch.max_q_len == 1 and attention_talk_splits > 1:
                seen = batch.max_kv_len if not window else min(batch.max_kv_len, window + 32)
                splits = max(1, min(attention_talk_splits, (2 * sm_count(q.device)) // batch.num_requests, (seen // 32 + 1) // 2))
                if splits > 1:
                    part = workspace.get("attn_talk_part", (splits, t * num_heads, value_dim + 2), torch.float32)
            _call(lib, lib.tllm_attention_talk_mma, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
                  block_table.shape[1], _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(mix_log2), _ptr(sink), _ptr(gate),
                  0 if gate is None else gate.stride(0), _ptr(out), 1 if out.dtype == torch.float32 else 0, t,
                  batch.num_requests, batch.max_q_len, num_heads, num_kv_heads, k_cache.shape[2], ll(k_cache.stride(0)),
                  ll(k_cache.stride(1)), ll(v_cache.stride(0)), ll(v_cache.stride(1)), int(window or 0), splits, _ptr(part),
                  int(attention_talk_stages), _stream())
            return
    lib = build.load_library("attention_talk")
    _call(lib, lib.tllm_attention_talk, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
          block_table.shape[1], _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(mix), _ptr(sink), _ptr(gate),
          0 if gate is None else gate.stride(0), _ptr(out), 1 if out.dtype == torch.float32 else 0, batch.num_requests,
          batch.max_q_len, num_heads, num_kv_heads, key_dim, value_dim, k_cache.shape[2], ll(k_cache.stride(0)),
          ll(k_cache.stride(1)), ll(v_cache.stride(0)), ll(v_cache.stride(1)), int(window or 0), _code(q.dtype), _stream())


# ----------------------------------------------------------------------------- matrix products


EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SWIGLU, EPI_ATOMIC_F32 = 0, 1, 2, 3, 4
EPI_CL_ADD_F32, EPI_CL_ROPE_KV, EPI_CL_SWIGLU, EPI_CL_BF16 = 5, 6, 7, 8   # K slices reduced inside a thread-block cluster
_sm_count = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (cudaDevAttrMultiProcessorCount), read once per device:
    the slice counts below are sized to fill them."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if index not in _sm_count:
        _sm_count[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_count[index]


force_generic = False   # tests set this to compare the tensor-core kernels with the SIMT ones
split_k = os.environ.get("TLLM_SPLIT_K", "1") != "0"   # slices of K at decode (a switch for measurements)
# which products of few rows reduce their K slices inside a thread-block cluster instead of with float32
# atomics: 1 = residual add / plain store, 2 = Q/K/V with rotation and cache write, 4 = SiLU * up.
# Measured at the TinyLlama shape (decode, batch 8): 0 -> 1.109 ms, 6 -> 1.087 ms, 7 -> 1.185 ms per
# step: the fused epilogues save a kernel each, the cluster's barriers cost about as much as one.
cluster_mask = int(os.environ.get("TLLM_CLUSTER", "6"))
cluster_reduce = cluster_mask != 0
_status = {}


def status_word(device) -> torch.Tensor:
    """The device int in which a kernel records that one of its bounded waits expired."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


_STATUS_CODES = ("1 = TMA producer, 2 = MMA issuer, 3 = epilogue of a matrix product; 7 = TMA producer, "
                 "8 = MMA issuer, 9 = softmax of the tensor-core attention")


def raise_status(device, code: int) -> None:
    """Clears the device's status word and raises for the code that was read from it."""
    key = torch.device(device).index or 0
    if key in _status:
        _status[key].zero_()
    raise KernelError(f"a kernel on device {key} gave up waiting (code {code}: {_STATUS_CODES}); "
                      f"the step's output is not valid and was dropped")


def check_status() -> None:
    """Reads the status words (a device synchronisation) and raises if a kernel gave up a wait.
    The generation path does not call this: there the word travels with the sampled ids
    (`argmax` / `sample` with `status`)."""
    for key, t in _status.items():
        code = int(t.item())
        if code:
            raise_status(f"cuda:{key}", code)


def _tc_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    k = a.shape[1]
    return (not force_generic and a.dtype == torch.bfloat16 and k % 8 == 0 and a.stride(0) % 8 == 0 and
            a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _swap_splits(n: int, k: int, atomic_ok: bool) -> int:
    """How many slices of K a weight tile of 128 rows is cut into at decode: enough CTAs to have
    every SM stream weights, but at least four 64-wide blocks per slice.  (Measured: counts that fill
    the SMs more evenly but with fewer CTAs -- 9 instead of 10 slices of the down projection, 3 instead
    of 2 for gate/up -- made the step slower, not faster.)"""
    if not atomic_ok or not split_k:
        return 1
    row_tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    want = -(-sm_count() // row_tiles)
    return max(1, min(want, k_blocks // 4))


def _cluster_slices(n: int, k: int, limit: int = 8) -> int:
    """Slices of K per weight tile for the cluster kernel: 1, 2, 4 or 8, enough CTAs for every SM, at
    least four 64-wide blocks per slice."""
    s = _swap_splits(n, k, True)
    p = 1
    while p * 2 <= min(s, limit):
        p *= 2
    return p


def _cluster_call(epi, a, w, out, slices, positions=None, cos=None, sin=None, nq=0, nkv=0, hd=0, k_cache=None,
                  v_cache=None, slot_mapping=None):
    lib = build.load_library("linear_tc")
    m, k = a.shape
    page_size = page_stride = head_stride = 0
    if k_cache is not None:
        page_size, page_stride, head_stride = k_cache.shape[2], k_cache.stride(0), k_cache.stride(1)
    _call(lib, lib.tllm_linear_tc_cluster,
        _ptr(a), _ptr(w), _ptr(out), m, w.shape[0], k, a.stride(0), out.stride(0), epi, slices, _ptr(positions),
        _ptr(cos), _ptr(sin), nq, nkv, hd, _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), page_size,
        ctypes.c_longlong(page_stride), ctypes.c_longlong(head_stride), _ptr(status_word(a.device)), _stream())


def linear_rope_kv(h: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                   head_dim: int, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   slot_mapping: Optional[torch.Tensor]) -> bool:
    """Q/K/V projection with the rotation and the cache write in its epilogue (a cluster per weight tile
    for at most 128 tokens, 128 x 256 tiles of the product for more):
    the rotated queries go to the first num_heads*head_dim values of each `qkv` row, rotated keys and
    values straight into their pages (slot_mapping None: `w_qkv` holds the query rows only).  Returns
    False, having done nothing, where the fused kernel does not apply (then: linear + rope_kv_write)."""
    m = h.shape[0]
    if not ((cluster_mask & 2) and _tc_ok(h, w_qkv, qkv) and head_dim in ((16, 32, 64, 128) if m <= 128 else (64, 128)) and
            qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and w_qkv.is_contiguous() and
            (cos is None or cos.shape[1] * 2 == head_dim)):
        return False
    _need_cuda(h, w_qkv, qkv, positions, cos, sin, k_cache, v_cache, slot_mapping)
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    want = num_heads * head_dim + (0 if slot_mapping is None else 2 * num_kv_heads * head_dim)
    if w_qkv.shape != (want, h.shape[1]) or qkv.shape[0] != m or qkv.shape[1] < num_heads * head_dim:
        raise KernelError("linear_rope_kv: shapes do not fit")
    if slot_mapping is not None and (k_cache.dtype != torch.bfloat16 or k_cache.stride() != v_cache.stride() or
                                     k_cache.stride(3) != 1 or k_cache.stride(2) != head_dim):
        raise KernelError("linear_rope_kv: cache layout does not fit")
    _cluster_call(EPI_CL_ROPE_KV, h, w_qkv, qkv, _cluster_slices(want, h.shape[1]) if m <= 128 else 1, positions, cos, sin, num_heads,
                  num_kv_heads, head_dim, k_cache if slot_mapping is not None else None,
                  v_cache if slot_mapping is not None else None, slot_mapping)
    return True


# Up to this many tokens (and above 128, where the product runs as 128 x 256 tiles) the Q/K/V projection takes the
# kernel with rotation and cache write in its epilogue, whatever the sizes.  Between, a cluster of eight K slices hands
# round 8 x 128 x tokens float32 values per weight tile, and K slices added with float32 atomics plus the
# rotate-and-cache kernel are faster (ms per decode step at the TinyLlama sizes, 8 slices, fused / separate: 16 tokens
# 0.935 / 0.932, 24 1.059 / 1.063, 32 1.123 / 1.097, 64 1.576 / 1.518); with fewer slices the fused kernel stays
# (Llama-3-8B sizes, 4 slices, 8 layers: 32 tokens 1.326 / 1.428, 64 1.802 / 1.840).
qkv_fused_rows = int(os.environ.get("TLLM_QKV_FUSED_ROWS", "24"))


def fused_qkv_preferred(m: int, n: int, k: int) -> bool:
    return m <= qkv_fused_rows or m > 128 or _cluster_slices(n, k) < 8


# float32 products of at most 16 rows take a kernel of their own (one thread per output element, weights streamed
# through shared memory); False keeps the 64 x 64 tiles.  Both give the same bits (tests compare them).
linear_skinny = True


def prefers_split(a: torch.Tensor, w: torch.Tensor) -> bool:
    """True when `linear` would cut K into slices for this product if it may add into a float32
    output: few rows (decode), so few weight tiles that the SMs only fill when K is split too.
    A caller that wants a bfloat16 result then accumulates into a zeroed float32 buffer and lets the
    next kernel convert (silu_mul / rope_kv_write with consume/src)."""
    return _tc_ok(a, w, None) and a.shape[0] <= 128 and _swap_splits(w.shape[0], a.shape[1], True) > 1


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           cluster_slices: bool = False) -> None:
    """out = a . w^T (w is [N, K], rows contiguous).  `out` may be of a's dtype or float32;
    accumulate=True adds the product into a float32 `out`.  cluster_slices=True: a product of at most 128 rows
    that stores bfloat16 cuts K into slices that meet in a thread-block cluster (every SM streams weights; without
    it such a product has one CTA per 128 output columns, which walks all of K).  bfloat16 products run on the tensor
    cores (tcgen05) when K and the row stride of `a` are multiples of 8; float32 products, and
    the sizes TMA cannot take, run on the SIMT kernel."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or a.dtype != w.dtype or a.stride(1) != 1 or \
            out.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"linear: shapes or dtypes do not fit: a {tuple(a.shape)} {a.dtype}, "
                          f"w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)} {out.dtype}")
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("linear: accumulation needs a float32 output")
        mode = OUT_ACC
    elif out.dtype == a.dtype:
        mode = OUT_SAME
    elif out.dtype == torch.float32:
        mode = OUT_F32
    else:
        raise KernelError(f"linear: output dtype {out.dtype} does not fit input dtype {a.dtype}")
    if _tc_ok(a, w, out):
        lib = build.load_library("linear_tc")
        epi = {OUT_SAME: EPI_BF16, OUT_F32: EPI_F32, OUT_ACC: EPI_ADD_F32}[mode]
        swap, splits = 0, 1
        if m <= 128:
            swap = 1
            if ((cluster_mask & 1) and mode in (OUT_ACC, OUT_SAME)) or (cluster_slices and split_k and mode == OUT_SAME):
                slices = _cluster_slices(n, k)
                if slices > 1:   # the slices of K meet in a cluster: one writer per element, no atomics
                    _cluster_call(EPI_CL_ADD_F32 if mode == OUT_ACC else EPI_CL_BF16, a, w, out, slices)
                    return
            splits = _swap_splits(n, k, atomic_ok=(mode == OUT_ACC))
            if splits > 1:
                epi = EPI_ATOMIC_F32
        _call(lib, lib.tllm_linear_tc, _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), out.stride(0), epi, swap,
                                       splits, _ptr(status_word(a.device)), _stream())
        return
    lib = build.load_library("linear_generic")
    _call(lib, lib.tllm_linear_generic, _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), out.stride(0),
                                        _code(a.dtype), mode, int(linear_skinny), _stream())


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, block: int, workspace,
                  act: str = "silu") -> None:
    """out = act(a Wg^T) * (a Wu^T) with Wg, Wu interleaved in `w_gate_up` in row blocks of `block`; act = silu or relu.
    With blocks of 128 and more than 128 rows the product and SiLU*up are one tensor-core kernel (SiLU only: another
    activation takes the product and the element-wise kernel)."""
    m = a.shape[0]
    n2 = w_gate_up.shape[0]
    if act != "silu":
        if prefers_split(a, w_gate_up):
            acc = workspace.get_zeroed("gate_up_f32", (m, n2))
            linear(a, w_gate_up, acc, accumulate=True)
            silu_mul(acc, out, block, consume=True, act=act)
            return
        gu = workspace.get("gate_up", (m, n2), a.dtype)
        linear(a, w_gate_up, gu)
        silu_mul(gu, out, block, act=act)
        return
    if _tc_ok(a, w_gate_up, out) and block == 128 and m > 128 and n2 % 256 == 0 and out.is_contiguous():
        _need_cuda(a, w_gate_up, out)
        lib = build.load_library("linear_tc")
        _call(lib, lib.tllm_linear_tc, _ptr(a), _ptr(w_gate_up), _ptr(out), m, n2, a.shape[1], a.stride(0),
                                       out.stride(0), EPI_SWIGLU, 0, 1, _ptr(status_word(a.device)), _stream())
        return
    if (cluster_mask & 4) and _tc_ok(a, w_gate_up, out) and block == 128 and m <= 128 and n2 % 256 == 0 and \
            out.stride(1) == 1 and w_gate_up.is_contiguous():
        # the gate tile, the up tile beside it and their K slices form one cluster; SiLU * up in its epilogue
        _need_cuda(a, w_gate_up, out)
        _cluster_call(EPI_CL_SWIGLU, a, w_gate_up, out, _cluster_slices(n2, a.shape[1], limit=4))
        return
    if prefers_split(a, w_gate_up):
        acc = workspace.get_zeroed("gate_up_f32", (m, n2))
        linear(a, w_gate_up, acc, accumulate=True)
        silu_mul(acc, out, block, consume=True)
        return
    gu = workspace.get("gate_up", (m, n2), a.dtype)
    linear(a, w_gate_up, gu)
    silu_mul(gu, out, block)


# ----------------------------------------------------------------------------- attention


attention_tc = os.environ.get("TLLM_ATTENTION_TC", "1") != "0"   # tcgen05 attention for prompt portions (a switch for measurements)


def _attention_splits(num_requests: int, max_q_len: int, group: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Slices of keys per (request, key/value head).  Decoded tokens (at most 16 rows) run as small
    CTAs: the fewest slices that give at least 256 CTAs of at most 11 tiles of 64 keys each, each slice
    at least two tiles, and no slice empty.  (Measured at context 2,048: batch 1 -> 16 slices, 8 -> 8,
    16 -> 4, 32 and 64 -> 3; "fill three CTAs per SM once" had picked 14 at batch 8 and 2 at batch 64 and
    was 5 to 7 % slower.)  Portions of prompts are sliced only when there are fewer CTAs than SMs."""
    if max_q_len * group <= 16:
        ctas = num_requests * num_kv_heads
        tiles = max(1, -(-max_kv_len // 64))
        most = max(1, tiles // 2)
        pick = most
        for s in range(1, most + 1):
            if ctas * s >= 256 and -(-tiles // s) <= 11:
                pick = s
                break
        per_slice = -(-tiles // pick)
        return -(-tiles // per_slice)
    ctas = num_requests * (-(-max_q_len * group // 64)) * num_kv_heads
    sms = sm_count()
    if ctas >= sms:
        return 1
    return max(1, min(-(-2 * sms // ctas), max_kv_len // 256))


# Decoded tokens with one warp per 64-key tile (slices of four tiles, all of a slice's copies in flight at once, one
# block barrier instead of one per tile): taken when it gives this many CTAs.  Measured at the TinyLlama sizes,
# context 2,048, against the kernel that walks a slice tile by tile with four warps per tile (ms per step): batch 4
# 0.754 / 0.778, 8 0.810 / 0.826, 16 0.938 / 0.942; outside the range it loses: batch 1 0.724 / 0.716 (32 CTAs),
# batch 32 1.193 / 1.124 (1,024 CTAs).  TLLM_DECODE_WIDE=0 turns it off (a switch for measurements).
decode_wide_ctas = (96, 640) if os.environ.get("TLLM_DECODE_WIDE", "1") != "0" else (1, 0)
# ... and its 2 to 8 slices of a (request, key/value head) as one thread-block cluster that merges them over
# distributed shared memory, in place of partial results in global memory and a merging kernel behind it, while the
# CTAs are at most 1.75 per SM: a cluster starts only when all its CTAs find room at once, and past that count whole
# clusters wait for a second round (ms per step with / without, context 2,048: batch 4 0.744 / 0.753, 6 0.774 / 0.777,
# 8 0.800 / 0.811, but 9 0.871 / 0.829, 12 0.931 / 0.872, 16 0.973 / 0.940; the kernel that walks a slice tile by tile
# gains nothing from it at any batch: 64 1.547 / 1.506, 32 1.080 / 1.085, 24 1.084 / 1.063).  TLLM_DECODE_CLUSTER=0 turns it off.
decode_cluster_merge = os.environ.get("TLLM_DECODE_CLUSTER", "1") != "0"


def _cluster_merge(num_requests: int, num_kv_heads: int, splits: int) -> bool:
    return decode_cluster_merge and 2 <= splits <= 8 and num_requests * num_kv_heads * splits * 4 <= 7 * sm_count()


def _wide_splits(num_requests: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Slices of four tiles for the kernel with one warp per tile, or 0 where it is not taken."""
    splits = -(-max(1, -(-max_kv_len // 64)) // 4)
    lo, hi = decode_wide_ctas
    ctas = num_requests * num_kv_heads * splits
    if lo <= ctas <= hi:
        return splits
    # fewer CTAs than that: only where the slices then merge inside a cluster, which saves the merge kernel
    # (batch 1 at context 2,048: 0.684 ms per step against 0.714, batch 2 0.707 against 0.732)
    return splits if ctas < lo and hi > 0 and _cluster_merge(num_requests, num_kv_heads, splits) else 0


# The attention of the 32-bit path runs eight warps per (token, head) or one warp per (token, key/value head, four query
# heads), by the number of pairs; both give the same bits.  True / False force one of them, 2 the plainest form (one
# warp per pair); tests compare the three.
generic_attention_split = None


split_mixed_attention = os.environ.get("TLLM_SPLIT_MIXED_ATTENTION", "1") != "0"   # (a switch for measurements)


class _SubBatch:
    """Requests [lo, hi) of a step's batch, for a kernel that takes a run of the per-request tables."""

    def __init__(self, batch, lo: int, hi: int, max_q_len: int):
        self.cu_q = batch.cu_q[lo: hi + 1]
        self.q_start = batch.q_start[lo: hi]
        self.num_requests = hi - lo
        self.max_q_len = max_q_len
        self.max_kv_len = batch.max_kv_len
        self.token_request = batch.token_request
        self.positions = batch.positions
        self.num_leading_decodes = 0


def paged_attention(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, block_table: torch.Tensor, batch, out: torch.Tensor, scale: float,
                    window: Optional[int] = None, workspace=None) -> None:
    """Attention of every token of the step (queries in the first num_heads*head_dim values of each
    `qkv` row) over its request's pages.  `batch` carries the step's metadata: token_request and
    positions per token; cu_q, q_start per request; num_requests, max_q_len, max_kv_len.
    bfloat16 runs on the tensor-core kernel compiled for this head size (it needs `workspace` for the
    partial results when it slices the keys); float32 on the SIMT kernel."""
    _need_cuda(qkv, k_cache, v_cache, block_table, out)
    _i32(block_table, "block_table")
    t = qkv.shape[0]
    if out.shape != (t, num_heads * head_dim) or not out.is_contiguous() or out.dtype != qkv.dtype or \
            k_cache.dtype != qkv.dtype or k_cache.stride() != v_cache.stride() or k_cache.stride(3) != 1 or \
            k_cache.stride(2) != head_dim or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError("paged_attention: shapes or dtypes do not fit")
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    if qkv.dtype == torch.bfloat16 and not force_generic and attention_tc and head_dim in ATTENTION_TC_HEAD_DIMS and \
            not window and batch.max_q_len * group >= 128 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and \
            k_cache.is_contiguous() and v_cache.is_contiguous():
        # portions of prompts: 128 rows of (token, head of the group) per CTA on the tcgen05 tensor cores
        lib = build.load_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
        if lib.tllm_attention_tc_fits(num_heads, num_kv_heads, head_dim, page_size, 0):
            lead = getattr(batch, "num_leading_decodes", 0)
            if 0 < lead < batch.num_requests and group <= 16 and split_mixed_attention:
                # Decoded tokens beside portions, the decoded ones first (as the scheduler lays a step out): a CTA of
                # 128 rows would walk a whole context for the one token of a request.  They go to the decode kernel,
                # the rest to this one: two launches over two runs of the same tables.
                paged_attention(qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache, block_table[:lead],
                                _SubBatch(batch, 0, lead, 1), out, scale, window, workspace)
                paged_attention(qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache, block_table[lead:],
                                _SubBatch(batch, lead, batch.num_requests, batch.max_q_len), out, scale, window, workspace)
                return
            _call(lib, lib.tllm_attention_tc,
                _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]),
                _ptr(block_table), block_table.shape[1], _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(out), t,
                batch.num_requests, batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size,
                ctypes.c_float(scale), _ptr(status_word(qkv.device)), _stream())
            return
    if qkv.dtype == torch.bfloat16 and not force_generic and head_dim % 16 == 0 and 16 <= head_dim <= 256 and \
            qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        lib = build.load_library("attention_mma", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
        splits, wide = 1, 0   # wide: bit 0 = one warp per tile, bit 1 = the slices merge inside a cluster
        if workspace is not None:
            splits = _attention_splits(batch.num_requests, batch.max_q_len, group, num_kv_heads, batch.max_kv_len)
            if batch.max_q_len * group <= 16:
                wide_splits = _wide_splits(batch.num_requests, num_kv_heads, batch.max_kv_len) \
                    if lib.tllm_attention_mma_wide_fits() else 0
                if wide_splits:
                    splits, wide = wide_splits, (3 if _cluster_merge(batch.num_requests, num_kv_heads, wide_splits) else 1)
        scratch = None
        if splits > 1 and not wide & 2:
            scratch = workspace.get("attention_partials", (t * num_heads * splits * (head_dim + 2),), torch.float32)
        _call(lib, lib.tllm_attention_mma,
            _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(out), t, batch.num_requests, batch.max_q_len, num_heads,
            num_kv_heads, head_dim, page_size, ctypes.c_longlong(k_cache.stride(0)),
            ctypes.c_longlong(k_cache.stride(1)), ctypes.c_float(scale), int(window or 0), splits, _ptr(scratch),
            wide, int(batch.max_kv_len), _stream())
        return
    lib = build.load_library("attention_generic")
    _call(lib, lib.tllm_paged_attention_generic,
        _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(batch.token_request), _ptr(batch.positions), _ptr(out), t, num_heads, num_kv_heads, head_dim,
        page_size, ctypes.c_longlong(k_cache.stride(0)), ctypes.c_longlong(k_cache.stride(1)),
        ctypes.c_float(scale), int(window or 0), _code(qkv.dtype),
        -1 if generic_attention_split is None else int(generic_attention_split), _stream())


# bfloat16 attention with several score maps per head on the tensor cores (False: the CUDA-core kernel; for measurements)
attention_maps_tc = os.environ.get("TLLM_ATTENTION_MAPS_TC", "1") != "0"


# Decoded tokens alone in a step, up to this many (token, head, map) pairs: the CUDA-core kernel, which gives eight
# warps to every pair and so walks a pair's keys eight tiles at a time, instead of the tensor-core kernel, whose one
# CTA per (request, key row) walks them tile after tile (0: always the tensor-core kernel; a switch for measurements).
attention_maps_decode_pairs = int(os.environ.get("TLLM_ATTENTION_MAPS_DECODE_PAIRS", "0"))
# Decoded tokens alone in a step: the tensor-core kernel cuts a row tile's key tiles into up to this many runs when its
# grid (requests x key rows) would leave SMs idle; the runs' sums are joined by a second kernel (0 or 1: one run).
attention_maps_splits = int(os.environ.get("TLLM_ATTENTION_MAPS_SPLITS", "16"))


def paged_attention_maps(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, maps: int, key_dim: int, value_dim: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor, batch,
                         out: torch.Tensor, scale: float, window: Optional[int] = None,
                         chunk: Optional[int] = None, sink: Optional[torch.Tensor] = None, workspace=None) -> None:
    """Attention with `maps` score maps per head over the same values, key rows of key_dim and value rows of
    value_dim values: query rows [head][map][key_dim] at the front of each `qkv` row, k_cache
    [pages, num_kv_heads * maps, page_size, key_dim], v_cache [pages, num_kv_heads, page_size, value_dim]; out
    [T, num_heads * maps * value_dim] in the cache's dtype or float32.  `chunk`: a key is visible only inside the
    query's chunk of that many positions (counted from position 0).  `sink` (float32 [num_heads]): a learned score
    per head whose exponential joins the softmax's denominator; it stands for no key and has no value.
    `batch`: token_request and positions per token
    (the CUDA-core kernel); cu_q, q_start per request, num_requests, max_q_len (the tensor-core kernel).
    bfloat16 with a float32 output and sizes that are multiples of 16 runs on the tensor cores, everything else on
    the CUDA cores in 32-bit.  `workspace` (the step's named buffers): lets a step of decoded tokens cut the keys of a
    row tile into runs that separate CTAs walk (needs batch.max_kv_len, an upper bound of the contexts)."""
    _need_cuda(qkv, k_cache, v_cache, block_table, out, sink)
    _i32(block_table, "block_table")
    t = qkv.shape[0]
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != num_heads or not sink.is_contiguous()):
        raise KernelError("paged_attention_maps: the sink is one float32 per head")
    if out.shape != (t, num_heads * maps * value_dim) or not out.is_contiguous() or \
            out.dtype not in (qkv.dtype, torch.float32) or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or \
            k_cache.stride(3) != 1 or k_cache.stride(2) != key_dim or k_cache.shape[1] != num_kv_heads * maps or \
            k_cache.shape[3] != key_dim or v_cache.stride(3) != 1 or v_cache.stride(2) != value_dim or \
            v_cache.shape[1] != num_kv_heads or v_cache.shape[3] != value_dim or k_cache.shape[2] != v_cache.shape[2]:
        raise KernelError("paged_attention_maps: shapes or dtypes do not fit")
    few = getattr(batch, "max_q_len", 0) == 1 and t * num_heads * maps <= attention_maps_decode_pairs
    if qkv.dtype == torch.bfloat16 and out.dtype == torch.float32 and not force_generic and attention_maps_tc and \
            not few and scale > 0 and key_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= key_dim <= 256 and 16 <= value_dim <= 256 and \
            qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        # bfloat16: the tensor-core kernel compiled for this pair of sizes (prompt portions and decoded tokens alike)
        lib = build.load_library("attention_maps_mma", flags=(f"-DTLLM_HEAD_DIM={key_dim}", f"-DTLLM_VALUE_DIM={value_dim}"))
        splits, part = 1, None
        if workspace is not None and batch.max_q_len == 1 and attention_maps_splits > 1 and num_heads // num_kv_heads <= 64:
            seen = batch.max_kv_len if not window else min(batch.max_kv_len, window + 64)
            if chunk:
                seen = min(seen, chunk)
            ctas = batch.num_requests * num_kv_heads * maps
            splits = max(1, min(attention_maps_splits, (4 * sm_count(qkv.device)) // ctas, (seen // 64 + 1) // 2))
            if splits > 1:
                part = workspace.get("attn_maps_part", (splits, t * num_heads * maps, value_dim + 2), torch.float32)
        _call(lib, lib.tllm_attention_maps_mma,
              _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
              _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(out), t, batch.num_requests, batch.max_q_len, num_heads,
              num_kv_heads, maps, key_dim, value_dim, k_cache.shape[2], ctypes.c_longlong(k_cache.stride(0)),
              ctypes.c_longlong(k_cache.stride(1)), ctypes.c_longlong(v_cache.stride(0)),
              ctypes.c_longlong(v_cache.stride(1)), ctypes.c_float(scale), int(window or 0), int(chunk or 0), _ptr(sink),
              splits, _ptr(part), _stream())
        return
    lib = build.load_library("attention_generic")
    _call(lib, lib.tllm_paged_attention_maps,
          _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
          _ptr(batch.token_request), _ptr(batch.positions), _ptr(out), t, num_heads, num_kv_heads, maps, key_dim,
          value_dim, k_cache.shape[2], ctypes.c_longlong(k_cache.stride(0)), ctypes.c_longlong(k_cache.stride(1)),
          ctypes.c_longlong(v_cache.stride(0)), ctypes.c_longlong(v_cache.stride(1)), ctypes.c_float(scale),
          int(window or 0), int(chunk or 0), _code(qkv.dtype), 1 if out.dtype == torch.float32 else 0,
          -1 if generic_attention_split is None else int(generic_attention_split), _ptr(sink), _stream())


def attention_tc_timing(head_dim: int = 64) -> Optional[dict]:
    """Cycles that the roles of the prompt-attention kernel's first CTA spent per phase since the last call, or
    None if the kernel was not built with TLLM_NVCC_FLAGS_ATTENTION_TC=-DTLLM_ATT_TIMING=1."""
    if head_dim not in ATTENTION_TC_HEAD_DIMS:
        return None
    lib = build.load_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
    if not hasattr(lib, "tllm_attention_tc_timing"):
        return None
    out = (ctypes.c_ulonglong * 16)()
    lib.tllm_attention_tc_timing(out)
    names = ["softmax: wait S", "softmax: S to registers", "softmax: max, exp2, sum", "softmax: P to tensor memory",
             "(unused)", "softmax: vote, store wait", "softmax: fence, arrive", "rescales of O",
             "qk: wait K", "qk: wait S buffer", "pv: wait V", "qk: issue", "tma: wait free stage", "tma: issue",
             "pv: wait P", "pv: issue"]
    return {n: int(v) for n, v in zip(names, out) if n != "(unused)"}


# ----------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """out[i] = first maximum of row i.  `status`: the device's status word; `out` then holds n + 1
    ints and out[n] receives the word, so that it travels to the host with the ids."""
    _need_cuda(logits, out, status)
    _i32(out, "out")
    _i32(status, "status")
    n, v = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or out.numel() != n + (status is not None):
        raise KernelError("argmax: logits must be contiguous float32 [n, V] and out int32 [n] (n + 1 with a status word)")
    lib = build.load_library("sampling")
    _call(lib, lib.tllm_argmax, _ptr(logits), _ptr(out), n, v, _ptr(status), _stream())


def sample(logits: torch.Tensor, work: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor, out: torch.Tensor,
           status: Optional[torch.Tensor] = None) -> None:
    """Temperature -> top-k -> top-p -> multinomial per row; rows with temperature <= 0 are greedy.
    `work` is float32 scratch of at least n*V elements; seeds and counters are int64 (read as
    unsigned 64-bit).  `status` as for argmax."""
    _need_cuda(logits, work, temperature, top_k, top_p, seeds, counters, out, status)
    _i32(top_k, "top_k")
    _i32(out, "out")
    _i32(status, "status")
    n, v = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or work.dtype != torch.float32 or \
            work.numel() < n * v or temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or \
            seeds.dtype != torch.int64 or counters.dtype != torch.int64 or out.numel() != n + (status is not None) or \
            any(x.numel() != n for x in (temperature, top_k, top_p, seeds, counters)):
        raise KernelError("sample: shapes or dtypes do not fit")
    lib = build.load_library("sampling")
    _call(lib, lib.tllm_sample, _ptr(logits), _ptr(work), n, v, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                _ptr(seeds), _ptr(counters), _ptr(out), _ptr(status), _stream())


ALL_LIBRARIES = ("elementwise", "linear_generic", "linear_tc", "attention_generic", "attention_prep", "recurrence",
                 "linear_attention", "delta_rule", "head_linear", "window_attention", "attention_talk", "moe", "sampling")


ATTENTION_HEAD_DIMS = (16, 32, 48, 64, 128)   # head sizes `build_all` compiles ahead; others compile on first use
ATTENTION_TC_HEAD_DIMS = (64, 128)            # head sizes the tcgen05 prompt-attention kernel is written for
ATTENTION_MAPS_DIMS = ((64, 128), (128, 128), (256, 192))           # (key size, value size) pairs of the multi-map kernel compiled ahead


WINDOW_ATTENTION_DIMS = ((64, 128),)   # (key size, value size) pairs of the window attention built ahead; others on first use


ATTENTION_TALK_DIMS = ((128, 128),)    # (key size, value size) pairs of the mixed-scores tensor-core kernel compiled ahead


def build_all(verbose: bool = True):
    """Compiles every library (what `__graft_entry__.build()` calls); returns their paths."""
    paths = [build.compile_library(n, verbose=verbose) for n in ALL_LIBRARIES]
    paths += [build.compile_library("attention_mma", flags=(f"-DTLLM_HEAD_DIM={hd}",), verbose=verbose)
              for hd in ATTENTION_HEAD_DIMS]
    paths += [build.compile_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={hd}",), verbose=verbose)
              for hd in ATTENTION_TC_HEAD_DIMS]
    paths += [build.compile_library("attention_maps_mma", flags=(f"-DTLLM_HEAD_DIM={kd}", f"-DTLLM_VALUE_DIM={vd}"), verbose=verbose)
              for kd, vd in ATTENTION_MAPS_DIMS]
    paths += [build.compile_library("attention_talk_mma", flags=(f"-DTLLM_HEAD_DIM={kd}", f"-DTLLM_VALUE_DIM={vd}"), verbose=verbose)
              for kd, vd in ATTENTION_TALK_DIMS]
    paths += [build.compile_library("window_attention_mma", flags=(f"-DTLLM_HEAD_DIM={kd}", f"-DTLLM_VALUE_DIM={vd}"), verbose=verbose)
              for kd, vd in WINDOW_ATTENTION_DIMS]
    return paths
