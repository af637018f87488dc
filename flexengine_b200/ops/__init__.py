"""The kernels as Python functions over CUDA tensors.

Every function here launches hand-written CUDA from ``csrc/`` on the current stream;
the only library calls are bfloat16 matrix products (cuBLAS through ``torch.mm``), where
the reference uses a library too (src/flexengine/inference/models/qwen2.py:99-101,129-135).
There is no CPU path: tensors must be on a CUDA device, and a missing or unbuildable
kernel library raises.

Conventions: activations are float32 (true 32-bit path) or bfloat16; the residual stream,
norm weights, biases and logits are float32; index tensors are int32.
"""
from __future__ import annotations

import torch

from . import library

# Arguments go to the entry points as plain Python values: the loader has given every entry point the parameter
# types of its C declaration (ops/library.py), so ctypes converts them itself, and refuses a call whose number of
# arguments or kinds of values do not fit.  These names say which C type a value is meant for.
_c_int, _c_ll, _c_float = int, int, float

# The library's bfloat16 products add the partial sums of a split K up in float: its default allows bfloat16 there, which
# costs two to four times the error of one bfloat16 rounding at K of a few thousand (measured against the
# weight-streaming kernel of this package, whose results are the float sums rounded once).
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

_status: dict = {}
launches = 0          # kernels of this package launched so far (library matrix products not counted)


def _core():
    return library.load("core")


def _ptr(t):
    return t.data_ptr() if t is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle; asked for at every launch, so by the shortest way there is."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise TypeError(f"kernels take float32 or bfloat16, not {dtype}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flexengine_b200.ops runs on CUDA tensors only; there is no CPU path")


def _run(lib, name: str, *args) -> None:
    global launches
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed: {lib.fe_last_error().decode()}")
    launches += 1


def status_word(device) -> torch.Tensor:
    """The device word in which kernels record a guarded fault (bad token, page or slot)."""
    word = _status.get(device)                     # asked for at every launch: the device object itself is the key
    if word is None:
        key = str(torch.device(device))
        if key not in _status:
            with torch.inference_mode(False):      # a plain tensor, writable from any mode
                _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
        word = _status[device] = _status[key]
    return word


STATUS_BITS = ((1, "token id out of range"), (2, "page id out of range"), (4, "cache slot out of range"),
               (8, "a bounded wait ran out"))


def describe_status(value: int) -> str:
    """What the bits of a status word say, in words."""
    return ", ".join(n for bit, n in STATUS_BITS if value & bit) or f"unknown bits {value}"


def check_status(device) -> None:
    """Synchronises; raises if a kernel met an index it had to skip since the last check."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        raise RuntimeError("kernel status: " + describe_status(value))


# ------------------------------------------------------------------------------------------------
def embedding(token_ids, table, scale=1.0, streams=None):
    """float32 residual rows [T, H] = table[token_ids]; with ``scale`` or ``streams``, rows times ``scale`` as
    [streams, T, H] (every copy the same), or [T, H] for ``streams`` None."""
    _need_cuda(token_ids, table)
    T, (V, H) = token_ids.numel(), table.shape
    if scale != 1.0 or streams is not None:
        copies = 1 if streams is None else int(streams)
        out = torch.empty((copies, T, H), dtype=torch.float32, device=table.device)
        _run(_core(), "fe_embedding_streams", _ptr(token_ids), _ptr(table), _ptr(out), _c_int(T), _c_int(H), _c_int(V), _c_float(scale),
             _c_int(copies), _c_int(_code(table.dtype)), _ptr(status_word(table.device)), _stream())
        return out[0] if streams is None else out
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _run(_core(), "fe_embedding", _ptr(token_ids), _ptr(table), _ptr(out), _c_int(T), _c_int(H), _c_int(V),
         _c_int(_code(table.dtype)), _ptr(status_word(table.device)), _stream())
    return out


def carry_tokens(token_ids, rows, sources, previous):
    """token_ids[rows[i]] = previous[sources[i]] where rows[i] >= 0 (all int32, in place): what the
    step before sampled becomes this step's input without a round trip through the host."""
    _need_cuda(token_ids, rows, sources, previous)
    if previous.dtype != torch.int32 or token_ids.dtype != torch.int32:
        raise TypeError("carry_tokens: int32 tensors")
    _run(_core(), "fe_carry_tokens", _ptr(token_ids), _ptr(rows), _ptr(sources), _ptr(previous), _c_int(rows.numel()),
         _c_int(token_ids.numel()), _c_int(previous.numel()), _ptr(status_word(token_ids.device)), _stream())


UPCOMING_MAX_ROWS = 16            # a step of this many tokens or fewer leaves the memory system idle between products
UPCOMING_BYTES_MERGE = 16 << 20   # the same for the merge kernel of decode attention, ahead of the output projection
UPCOMING_TAIL_BYTES = 16 << 20    # what the blocks of a weight-streaming product ask into L2 of the next matrix as they end
UPCOMING_BYTES = 10 << 20         # how much of the next weight matrix a norm asks into L2 ahead of its product: what the
                                  # memory system delivers while the norm runs (8-12 MB measured best on the 7B shape)


def _upcoming(tensor, rows: int, limit: int = UPCOMING_BYTES):
    """(pointer, bytes) of the start of ``tensor`` for a kernel's prefetching blocks; nothing for large steps."""
    if tensor is None or rows > UPCOMING_MAX_ROWS or not tensor.is_cuda:
        return None, 0
    return _ptr(tensor), _c_ll(min(tensor.numel() * tensor.element_size(), limit))


def _post_norm(residual, delta, post, weight, eps, out, rows, n_out, extra=None):
    """One launch of the kernel for branches that end in a norm of their own (csrc/post_norm.cu); see its callers."""
    T, H = residual.shape
    post_w, post_eps, bias = post if post is not None else (None, 0.0, None)
    _need_cuda(residual, delta, weight, rows, post_w, bias, extra)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    for vector in (weight, post_w, bias):
        if vector is not None and (vector.dtype != torch.float32 or vector.numel() != H):
            raise TypeError("norm weights and biases are float32 vectors of the stream's width")
    if delta is not None and (delta.dtype not in (torch.float32, out.dtype) or tuple(delta.shape) != (T, H) or not delta.is_contiguous()):
        raise ValueError("a branch output is contiguous, shaped like the residual, float32 or in the compute dtype")
    extra_cols = 0
    if extra is not None:
        if extra.dtype != torch.float32 or extra.dim() != 2 or extra.shape[0] != T or not extra.is_contiguous():
            raise ValueError("extra rows are contiguous float32 [T, columns]")
        extra_cols = extra.shape[1]
    _run(_core(), "fe_post_norm", _ptr(residual), _ptr(delta), _c_int(_code(delta.dtype) if delta is not None else 0), _ptr(bias),
         _ptr(post_w), _c_float(post_eps), _ptr(weight), _c_float(eps), _ptr(out), _c_ll(out.stride(0)), _ptr(rows), _c_int(n_out),
         _c_int(H), _ptr(extra), _c_int(extra_cols), _c_int(T), _c_int(_code(out.dtype)), _stream())
    return out


def residual_concat(residual, delta, extra, out_dtype, post=None):
    """residual += delta (through a norm of its own with ``post`` = (weight, eps, bias still to add)), then the rows
    [residual | extra] in ``out_dtype``: what a product reads that re-enters the stream from the stream and other float32
    rows of the same tokens."""
    T, H = residual.shape
    out = torch.empty((T, H + extra.shape[1]), dtype=out_dtype, device=residual.device)
    return _post_norm(residual, delta, post, None, 0.0, out, None, T, extra=extra)


def scale_softcap(logits, scale, cap):
    """logits <- cap * tanh(logits * scale / cap) in place (cap 0: logits * scale); float32."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise TypeError("scale_softcap: logits are contiguous float32")
    _run(_core(), "fe_scale_softcap", _ptr(logits), _c_ll(logits.numel()), _c_float(scale), _c_float(cap), _stream())
    return logits


def add_rmsnorm(residual, delta, weight, eps, out_dtype, rows=None, upcoming=None, post=None):
    """Fused residual add + RMSNorm.  rows=None: residual += delta in place (all rows) and every row
    is normalised; rows given: only those rows are read (residual[rows] + delta[rows]), nothing is
    written back.  ``upcoming``: the weight matrix that the next kernel streams; in a decode step extra
    blocks of this kernel, which barely touches memory, ask for its start to be brought into L2.
    ``post`` = (weight, eps, bias or None): the branch output goes through a norm of its own on its way into the stream,
    w_b (delta + bias) / rms(delta + bias); delta may then be float32 whatever the compute dtype."""
    if post is not None and delta is not None:
        T, H = residual.shape
        n_out = T if rows is None else rows.numel()
        out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
        return _post_norm(residual, delta, post, weight, eps, out, rows, n_out)
    _need_cuda(residual, delta, weight, rows)
    T, H = residual.shape
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError("the residual stream and norm weights are float32")
    if delta is not None and (delta.dtype != out_dtype or delta.shape != residual.shape or not delta.is_contiguous()):
        raise ValueError("add_rmsnorm: delta must be contiguous, shaped like the residual, in the compute dtype")
    n_out = T if rows is None else rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
    _run(_core(), "fe_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(weight), _c_float(eps), _ptr(out), _ptr(rows),
         _c_int(n_out), _c_int(H), _c_int(T), _c_int(_code(out_dtype)), *_upcoming(upcoming, T), _stream())
    return out


FUSES_RESIDUAL_NORM = True      # linear(..., follow=) may end a branch: see Prenormed


class Prenormed:
    """Rows that are halfway through an RMSNorm, as the residual epilogue of the weight-streaming GEMM leaves them
    (csrc/gemm_skinny.cu): ``scaled`` = bfloat16(residual * norm weight), not yet divided by the rows' root mean
    square, and ``sumsq`` [tiles of 16 columns, 8], every tile's share of the rows' sums of squares.  The products
    that consume a norm (``linear``, ``linear_swiglu``, ``qkv_projection``) take it in place of a tensor and
    finish the norm in their own epilogue; where that kernel does not apply, ``materialize`` runs the norm
    kernel over the residual, which holds the sum already."""
    __slots__ = ("scaled", "sumsq", "eps", "residual", "weight")

    def __init__(self, scaled, sumsq, eps, residual, weight):
        self.scaled, self.sumsq, self.eps, self.residual, self.weight = scaled, sumsq, float(eps), residual, weight

    shape = property(lambda self: self.scaled.shape)
    dtype = property(lambda self: self.scaled.dtype)
    device = property(lambda self: self.scaled.device)

    def materialize(self):
        return add_rmsnorm(self.residual, None, self.weight, self.eps, self.scaled.dtype)


def _rows_and_scale(x):
    """(tensor, sumsq pointer, tiles, eps) of an input of the weight-streaming kernel for up to 8 rows."""
    if isinstance(x, Prenormed):
        return x.scaled, _ptr(x.sumsq), _c_int(x.sumsq.shape[0]), _c_float(x.eps)
    return x, None, _c_int(0), _c_float(0.0)


def _fits(x, w) -> str:
    """Which weight-streaming kernel takes this product, if any: "skinny" (up to 8 rows) or ""."""
    return "skinny" if skinny_ok(x.scaled if isinstance(x, Prenormed) else x, w) else ""


def gemm_fp32(x, w, bias=None):
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _run(_core(), "fe_gemm_fp32", _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _stream())
    return out


def linear(x, w, bias=None, out_float32=False, follow=None, upcoming=None):
    """y = x w^T (+ bias); x [M, K], w [N, K].  A float32 weight runs the true 32-bit product
    (CUDA cores, no reduced-precision mode) whatever the activation dtype; a bfloat16 weight
    runs on tensor cores with float32 accumulation.

    ``follow`` = (residual, norm weight, eps): the product ends a branch of a layer; its result is to be added to
    the float32 residual stream [M, N] and an RMSNorm reads the sum next.  Where the weight-streaming kernel runs (a
    decode step), it does both in its epilogue and a ``Prenormed`` comes back; otherwise the plain product does,
    and the caller adds and normalises as usual.  ``upcoming``: the matrix that the kernel after this one streams;
    the weight-streaming kernel asks for its start to be brought into L2 as its blocks end."""
    kernel = _fits(x, w)
    if isinstance(x, Prenormed) and not kernel:
        x = x.materialize()
        kernel = _fits(x, w)
    rows = x.scaled if isinstance(x, Prenormed) else x
    _need_cuda(rows, w, bias)
    if follow is not None and bias is None and not out_float32 and kernel:
        residual, norm_weight, norm_eps = follow
        M, N = rows.shape[0], w.shape[0]
        if (residual.dtype == torch.float32 and tuple(residual.shape) == (M, N) and residual.is_contiguous()
                and norm_weight.dtype == torch.float32 and norm_weight.numel() == N):
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=rows.device)
            _rows, sumsq, tiles, eps = _rows_and_scale(x)
            table = torch.empty((-(-N // 16), 8), dtype=torch.float32, device=rows.device)
            _run(_bf16(), "fe_skinny_gemm_residual", _ptr(rows), _ptr(w), _ptr(residual), _ptr(norm_weight), _ptr(scaled),
                 _ptr(table), _c_int(M), _c_int(N), _c_int(rows.shape[1]), sumsq, tiles, eps,
                 *_upcoming(upcoming, M, UPCOMING_TAIL_BYTES), _stream())
            return Prenormed(scaled, table, norm_eps, residual, norm_weight)
    if kernel and w.dtype == torch.bfloat16:
        wide = out_float32 or bias is not None           # a bias is added in float32, before the one rounding
        y = skinny_gemm(x, w, EPI_F32 if wide else EPI_BF16, upcoming=upcoming)
        if bias is not None:
            y += bias
        return y if out_float32 or not wide else y.to(torch.bfloat16)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError(f"linear: shapes {tuple(x.shape)} x {tuple(w.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    if w.dtype == torch.float32:
        y = gemm_fp32(x if x.dtype == torch.float32 else x.float(), w, bias)
        return y if (out_float32 or x.dtype == torch.float32) else y.to(x.dtype)
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise TypeError(f"linear: weight {w.dtype} with activations {x.dtype}")
    wide = out_float32 or bias is not None           # a bias is added in float32, before the one rounding
    y = torch.mm(x, w.t(), out_dtype=torch.float32) if wide else torch.mm(x, w.t())
    if bias is not None:
        y += bias
    return y if out_float32 or not wide else y.to(torch.bfloat16)


SKINNY_MAX_ROWS = 8          # beyond this the library product is as fast or faster
SKINNY_QKV_MAX_ROWS = 8      # the fused projection + bias + rotation + cache write takes one 8-row tile of tokens
EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_GEGLU = 0, 1, 2, 5      # 5: the gated epilogue with the tanh form of GELU
EPI_RELU2 = 6                                               # relu(product)^2, no gate
GATED_EPILOGUES = {"silu": EPI_SWIGLU, "gelu_tanh": EPI_GEGLU}


def skinny_ok(x, w) -> bool:
    """Whether the weight-streaming kernel is used for this product: bfloat16, up to 8 rows (the
    kernel itself takes up to 16), K a multiple of 64."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS
            and x.shape[1] % 64 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(x, w, epilogue: int = EPI_BF16, upcoming=None):
    """x [M <= 16, K] (a tensor or a Prenormed) times w [N, K]^T by streaming w once; see csrc/gemm_skinny.cu."""
    x, sumsq, tiles, eps = _rows_and_scale(x)
    M, K = x.shape
    N = w.shape[0]
    if epilogue in (EPI_SWIGLU, EPI_GEGLU):
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    else:
        out = torch.empty((M, N), dtype=torch.float32 if epilogue == EPI_F32 else torch.bfloat16, device=x.device)
    _run(_bf16(), "fe_skinny_gemm_scaled", _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue),
         sumsq, tiles, eps, *_upcoming(upcoming, M, UPCOMING_TAIL_BYTES), _stream())
    return out


FUSED_NORM_MAX_ROWS = SKINNY_MAX_ROWS     # steps of up to this many tokens do their norms in the products' epilogues


TCGEN05_MIN_K = 1024
TCGEN05_MIN_ROWS = 1024      # measured: from about this many rows the fused kernel matches the library + activation


def tcgen05_ok(x, w) -> bool:
    """Whether the tcgen05 kernel is used for this product: bfloat16, many rows (prefill), K a multiple of 8 and
    long enough for the products of a tile to cover its epilogue (at K = 896 the library + activation is 10 % ahead,
    from K = 1,536 on the fused kernel is)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] >= TCGEN05_MIN_ROWS
            and x.shape[1] >= TCGEN05_MIN_K and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x, w, epilogue: int = EPI_BF16):
    """x [M, K] times w [N, K]^T on tcgen05 tensor cores (TMA operands, TMEM accumulator);
    epilogue EPI_BF16, EPI_SWIGLU, EPI_GEGLU or EPI_RELU2.  See csrc/gemm_tcgen05.cu."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
        raise TypeError("gemm_tcgen05 takes contiguous bfloat16 operands")
    out = torch.empty((M, N // 2 if epilogue in (EPI_SWIGLU, EPI_GEGLU) else N), dtype=torch.bfloat16, device=x.device)
    _run(_bf16(), "fe_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue),
         _ptr(status_word(x.device)), _stream())
    return out


def swiglu(gate_up, intermediate):
    _need_cuda(gate_up)
    T = gate_up.shape[0]
    if gate_up.shape[1] != 2 * intermediate or not gate_up.is_contiguous():
        raise ValueError("swiglu: input must be contiguous [T, 2 * intermediate]")
    out = torch.empty((T, intermediate), dtype=gate_up.dtype, device=gate_up.device)
    _run(_core(), "fe_swiglu", _ptr(gate_up), _ptr(out), _c_int(T), _c_int(intermediate),
         _c_int(_code(gate_up.dtype)), _stream())
    return out


def linear_swiglu(x, w, intermediate, upcoming=None):
    """silu(x Wg^T) * (x Wu^T) with w = [Wg; Wu] ([2I, K]); one kernel for a handful of rows."""
    kernel = _fits(x, w) if w.shape[0] == 2 * intermediate else ""
    if isinstance(x, Prenormed) and not kernel:
        x = x.materialize()
        kernel = _fits(x, w) if w.shape[0] == 2 * intermediate else ""
    if kernel == "skinny":
        return skinny_gemm(x, w, EPI_SWIGLU, upcoming=upcoming)
    if tcgen05_ok(x, w) and w.shape[0] == 2 * intermediate:
        return gemm_tcgen05(x, w, EPI_SWIGLU)
    return swiglu(linear(x, w), intermediate)


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def gated_activation(gate_up, intermediate, activation, bias=None, out_dtype=None):
    """act(gate) * up of rows [gate | up]; act "silu" or "gelu_tanh" (the tanh form of GELU), float arithmetic.  ``bias``
    (float32 [2 * intermediate]) is added to both first; the rows may then be a float32 product and ``out_dtype`` the
    compute dtype."""
    _need_cuda(gate_up, bias)
    T = gate_up.shape[0]
    if gate_up.shape[1] != 2 * intermediate or not gate_up.is_contiguous():
        raise ValueError("gated_activation: input must be contiguous [T, 2 * intermediate]")
    if activation not in GATE_ACTIVATIONS:
        raise ValueError(f"unknown gate activation {activation!r}; known: {sorted(GATE_ACTIVATIONS)}")
    if bias is not None or (out_dtype is not None and out_dtype != gate_up.dtype):
        out_dtype = out_dtype or gate_up.dtype
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != 2 * intermediate):
            raise ValueError("gated_activation: the bias is float32 [2 * intermediate]")
        out = torch.empty((T, intermediate), dtype=out_dtype, device=gate_up.device)
        _run(_core(), "fe_gated_activation_bias", _ptr(gate_up), _c_int(_code(gate_up.dtype)), _ptr(bias), _ptr(out), _c_int(T),
             _c_int(intermediate), _c_int(GATE_ACTIVATIONS[activation]), _c_int(_code(out_dtype)), _stream())
        return out
    out = torch.empty((T, intermediate), dtype=gate_up.dtype, device=gate_up.device)
    _run(_core(), "fe_gated_activation", _ptr(gate_up), _ptr(out), _c_int(T), _c_int(intermediate),
         _c_int(GATE_ACTIVATIONS[activation]), _c_int(_code(gate_up.dtype)), _stream())
    return out


def linear_gated(x, w, intermediate, activation):
    """act(x Wg^T) * (x Wu^T) with w = [Wg; Wu] ([2I, K]), act "silu" or "gelu_tanh": the weight-streaming kernel for a
    handful of rows and the tcgen05 kernel for a prompt's worth apply the gate's function in their epilogues; otherwise
    the product and the activation kernel."""
    if activation == "silu":
        return linear_swiglu(x, w, intermediate)
    if activation not in GATED_EPILOGUES:
        raise ValueError(f"unknown gate activation {activation!r}; known: {sorted(GATED_EPILOGUES)}")
    if isinstance(x, Prenormed):
        x = x.materialize()
    if w.shape[0] == 2 * intermediate:
        if _fits(x, w) == "skinny":
            return skinny_gemm(x, w, GATED_EPILOGUES[activation])
        if tcgen05_ok(x, w):
            return gemm_tcgen05(x, w, GATED_EPILOGUES[activation])
    return gated_activation(linear(x, w), intermediate, activation)


def qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache,
                        nq, nkv, d, page_size, src=None):
    """qkv [T, (nq + 2 nkv) d] = projection + bias, with the rotary encoding of the query and key heads;
    key and value heads are also written to their cache slots (slot_mapping None: no write).  The
    projection is ``qkv`` itself (rewritten in place) or ``src``, a float32 tensor of the same shape: a
    bfloat16 result is then rounded once, after bias and rotation."""
    _need_cuda(qkv, bias, positions, inv_freq, slot_mapping, k_cache, v_cache, src)
    T, width = qkv.shape
    if width != (nq + 2 * nkv) * d or not qkv.is_contiguous():
        raise ValueError("qkv_bias_rope_cache: qkv must be contiguous [T, (nq + 2 nkv) d]")
    if src is not None and (src.shape != qkv.shape or not src.is_contiguous() or src.dtype not in (torch.float32, qkv.dtype)):
        raise ValueError("qkv_bias_rope_cache: src must be contiguous, shaped like qkv, float32 or of its dtype")
    src_float = src is not None and src.dtype == torch.float32 and qkv.dtype != torch.float32
    if k_cache.dtype != qkv.dtype or tuple(k_cache.shape[1:]) != (nkv, page_size, d) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous():
        raise ValueError("qkv_bias_rope_cache: cache must be contiguous [pages, nkv, page_size, d] in the compute dtype")
    if bias is not None and bias.dtype != torch.float32:
        raise TypeError("biases are float32")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2):
        raise ValueError("inv_freq must be float32 [rot / 2]")
    num_slots = k_cache.shape[0] * page_size
    _run(_core(), "fe_qkv_bias_rope_cache", _ptr(qkv if src is None else src), _c_int(1 if src_float else 0), _ptr(qkv),
         _ptr(bias), _ptr(positions), _ptr(inv_freq), _c_int(rot),
         _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d),
         _c_int(page_size), _c_ll(num_slots), _c_int(_code(qkv.dtype)), _ptr(status_word(qkv.device)), _stream())


def qkv_projection(h, w, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size):
    """The query/key/value projection of an attention layer: h w^T + bias, rotary encoding of the
    query and key heads, new keys and values written to their cache slots (slot_mapping None: no
    write).  Returns qkv [T, (nq + 2 nkv) d].  For a handful of rows (decode) with the whole head
    rotated this is ONE kernel (csrc/gemm_skinny.cu); otherwise the product and the fused
    bias/rotation/cache-write kernel."""
    kernel = _fits(h, w)
    if isinstance(h, Prenormed) and not kernel:
        h = h.materialize()
        kernel = _fits(h, w)
    rows = h.scaled if isinstance(h, Prenormed) else h
    _need_cuda(rows, w, bias, positions, inv_freq, slot_mapping, k_cache, v_cache)
    whole_head = (inv_freq is not None and rot == d and k_cache.dtype == torch.bfloat16 and w.shape[0] == (nq + 2 * nkv) * d
                  and (bias is None or bias.dtype == torch.float32))
    if kernel == "skinny" and whole_head and d % 16 == 0 and rows.shape[0] <= SKINNY_QKV_MAX_ROWS:
        T = rows.shape[0]
        _rows, sumsq, tiles, eps = _rows_and_scale(h)
        out = torch.empty((T, w.shape[0]), dtype=torch.bfloat16, device=rows.device)
        _run(_bf16(), "fe_skinny_qkv", _ptr(rows), _ptr(w), _ptr(out), _ptr(bias), _ptr(positions), _ptr(inv_freq),
             _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(rows.shape[1]), _c_int(nq), _c_int(nkv),
             _c_int(d), _c_int(page_size), _c_ll(k_cache.shape[0] * page_size), sumsq, tiles, eps,
             _ptr(status_word(rows.device)), _stream())
        return out
    if isinstance(h, Prenormed):
        h = h.materialize()
    if h.dtype == torch.float32:
        qkv = linear(h, w)
        qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size)
        return qkv
    # the product stays float32 until bias and rotation are in, as in the fused kernel: a token's keys and values
    # are rounded once whichever path its step took
    product = linear(h, w, out_float32=True)
    qkv = torch.empty(product.shape, dtype=h.dtype, device=h.device)
    qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size,
                        src=product)
    return qkv


ATTENTION_SINK, ATTENTION_SIGMOID = 1, 2       # bits of the attention kernels' mode


def _attention_mode(sink: bool, sigmoid: bool) -> int:
    return (ATTENTION_SINK if sink else 0) | (ATTENTION_SIGMOID if sigmoid else 0)


def paged_attention_simt(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, token_request, T, nq, nkv, d,
                         page_size, scale, window, sink=False, sigmoid=False, head_bias=None):
    out = torch.empty((T, nq * d), dtype=k_cache.dtype, device=k_cache.device)
    mode = _attention_mode(sink, sigmoid)
    _run(_core(), "fe_paged_attention_simt", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start),
         _ptr(token_request), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size),
         _c_int(k_cache.shape[0]), _c_float(scale), _c_int(window), _c_int(mode), _c_int(_code(k_cache.dtype)),
         _ptr(status_word(k_cache.device)), _ptr(head_bias), _stream())
    return out


_scratch: dict = {}
_scratch_kept: list = []     # every scratch buffer ever handed out (see scratch())
_sm_count: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of ``device`` (the current CUDA device when None), as the driver reports them:
    the one number every launch heuristic here scales with (the kernels' own host code asks the same
    attribute through the helper in ``csrc/errors.cu``)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if index not in _sm_count:
        _sm_count[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_count[index]


def _bf16():
    return library.load("bf16")


def scratch(device, nbytes: int) -> torch.Tensor:
    """Scratch memory of at least ``nbytes`` bytes on ``device``, grown on demand.  A buffer that has been
    handed out is never freed: a CUDA graph captured with it keeps its address, and replays it long after a
    larger buffer has taken its place for new calls."""
    have = _scratch.get(device)
    if have is None or have.numel() < nbytes:
        key = str(torch.device(device))            # "cuda:0" and torch.device("cuda:0") share one buffer
        have = _scratch.get(key)
        if have is None or have.numel() < nbytes:
            with torch.inference_mode(False):
                have = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            _scratch_kept.append(have)
        for k in [k for k in _scratch if str(torch.device(k)) == key]:
            _scratch[k] = have
        _scratch[key] = _scratch[device] = have
    return have


DECODE_MAX_SPLITS = 256      # what the merge kernel of decode attention takes (fe_paged_decode_max_splits)


def decode_splits(requests: int, nkv: int, max_ctx_len: int, sms: int | None = None) -> int:
    """How many ways the keys of a request are split in decode.  Between half a round and one round of resident
    blocks (six blocks fit an SM; never more than a round: a few blocks over it would run alone after it): towards
    the full round when a split still has six tiles of 32 keys or more to walk, towards the half when splits
    would get short and the merge dominate; never a split shorter than two tiles, never more splits than the
    merge kernel takes (one request with one or two key/value heads at a very long context would ask for more)."""
    sms = sms or sm_count()
    tiles = max(1, -(-max_ctx_len // 32))
    pairs = max(1, requests * nkv)
    most = max(1, 6 * sms // pairs)               # rounded down: a few blocks over the round would run alone after it
    least = max(1, (3 * sms + pairs // 2) // pairs)
    want = min(most, max(least, tiles // 6), DECODE_MAX_SPLITS)
    return int(max(1, min(want, tiles // 2)))


def paged_decode_mma(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, requests, nq, nkv, d, page_size,
                     scale, window, splits, out=None, upcoming=None, sink=False, sigmoid=False, head_bias=None):
    """Tensor-core decode attention (one token per request), keys split ``splits`` ways.  ``upcoming``: the
    matrix that the next kernel streams (the output projection); extra blocks of the merge kernel ask for its
    start to be brought into L2."""
    if out is None:
        out = torch.empty((requests, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    lib = _bf16()
    need = lib.fe_paged_decode_scratch_bytes(_c_int(requests), _c_int(nq), _c_int(d), _c_int(splits))
    work = scratch(k_cache.device, need) if need else None
    _run(lib, "fe_paged_decode_mma_upcoming", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(out.stride(0)), _ptr(work),
         _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start),
         _c_int(requests), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _c_int(_attention_mode(sink, sigmoid)), _c_int(splits),
         *_upcoming(upcoming, requests, UPCOMING_BYTES_MERGE),
         _ptr(status_word(k_cache.device)), _ptr(head_bias), _stream())
    return out


DECODE_CLUSTER_MAX_SPLITS = 16       # blocks of one thread-block cluster (fe_paged_decode_cluster_max_splits)
DECODE_CLUSTER_MAX_TILES = 8         # a split of a cluster walks at most this many tiles of 32 keys ...
DECODE_CLUSTER_ONE_ROUND_MIN = 8     # ... and a cluster is cut down to fit one round only if this many splits remain
_CLUSTERS_RESIDENT: dict = {}


def clusters_resident(requests: int, nq: int, nkv: int, d: int, splits: int) -> int:
    """How many clusters of ``splits`` blocks of the decode kernel the device holds at once (asked of the driver once
    per shape): a cluster lives inside one of the GPU's processing clusters, so it is fewer than blocks / splits."""
    key = (requests, nq, nkv, d, splits)
    if key not in _CLUSTERS_RESIDENT:
        _CLUSTERS_RESIDENT[key] = int(_bf16().fe_paged_decode_cluster_resident(requests, nq, nkv, d, splits))
    return _CLUSTERS_RESIDENT[key]


def decode_cluster_splits(splits: int, max_ctx_len: int, clusters: int = 0, resident=None) -> int:
    """How many splits the cluster kernel takes for a step that ``decode_splits`` would split ``splits`` ways, or 0
    when the two-kernel form is the better one: a long context of a small batch, which wants more splits than a
    cluster holds, keeps them and the separate merge (batch 8 at 8,192 tokens: 3.53 against 3.59 ms a step of the 7B
    shape, at 16,384: 4.12 against 4.24; batch 1 at 16,384: 3.0 against 3.8).

    ``clusters``: how many clusters the step needs (requests x key/value heads); ``resident(s)``: how many clusters of
    s blocks the device holds at once.  A few clusters over one round run alone after it: 32 clusters of 15 or 16
    blocks, of which fewer than 32 fit, make a step 3.25 ms long where clusters of 8 to 14 make it 3.11 to 3.13, and
    64 clusters of 9 cost 4.07 ms where 64 of 8 cost 3.80.  So the count is cut down to the largest that fits one
    round, if that leaves eight splits or more; large batches, whose clusters of two to six blocks take several
    rounds anyway, keep their count (batch 64: three splits 4.88 ms, two 4.97)."""
    if splits <= 1:
        return 0
    most = min(splits, DECODE_CLUSTER_MAX_SPLITS)
    if splits > most and -(-max_ctx_len // 32) > most * DECODE_CLUSTER_MAX_TILES:
        return 0
    if resident is None or clusters <= 0:
        return most
    fit = next((s for s in range(most, 1, -1) if resident(s) >= clusters), 0)
    if fit >= min(most, DECODE_CLUSTER_ONE_ROUND_MIN):
        return fit
    return most if resident(most) > 0 else 0


def paged_decode_cluster(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, requests, nq, nkv, d, page_size,
                         scale, window, splits, out=None, sink=False, sigmoid=False, head_bias=None):
    """Decode attention with the splits of each (request, key/value head) as one thread-block cluster that merges
    its partial results through distributed shared memory: one launch, no scratch memory; splits <= 16."""
    if out is None:
        out = torch.empty((requests, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    _run(_bf16(), "fe_paged_decode_cluster", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(out.stride(0)), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]), _c_float(scale), _c_int(window),
         _c_int(_attention_mode(sink, sigmoid)), _c_int(splits), _ptr(status_word(k_cache.device)), _ptr(head_bias), _stream())
    return out


def paged_prefill_mma(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, T, requests, max_q_len, nq, nkv, d,
                      page_size, scale, window, sink=False, sigmoid=False, head_bias=None):
    """Tensor-core attention for portions of any length (decoded tokens are portions of one)."""
    out = torch.empty((T, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    _run(_bf16(), "fe_paged_prefill_mma", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(max_q_len), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _c_int(_attention_mode(sink, sigmoid)), _ptr(status_word(k_cache.device)), _ptr(head_bias),
         _stream())
    return out


def tcgen05_attention_ok(max_q_len, nq, nkv, d, lengths=None, starts=None, sms: int | None = None):
    """The tcgen05 prefill kernel takes head sizes 64 and 128, portions of any length: measured against the
    mma.sync kernel it is level on portions of a few tokens and ahead everywhere else, the more the longer the
    context.  Other head sizes go to the mma.sync kernel, and so does a step of many requests that bring a few
    tokens each to short contexts (``lengths`` and ``starts`` given): one tcgen05 block is resident on an SM and
    costs a few microseconds before its first tile, where several of the lighter blocks share an SM."""
    if d not in (64, 128):
        return False
    if lengths:
        group = nq // nkv
        blocks = nkv * sum(-(-n * group // 256) for n in lengths)
        rows = nkv * group * sum(lengths)
        longest = max(s + n for s, n in zip(starts, lengths))
        if blocks > (sms or sm_count()) and rows < 96 * blocks and longest <= 1024:
            return False
    return True


PREFILL_MAX_SPLITS = 32
PREFILL_TILES_PER_SPLIT = 4      # a split walks at least this many tiles of 64 keys
PREFILL_SPLIT_FROM_TILES = 16    # shorter walks are over before a second kernel could merge them


def prefill_splits(lengths, starts, nq, nkv, window=0, sms: int | None = None) -> int:
    """Into how many blocks the tcgen05 prefill kernel shares out the keys of each pair of row tiles.  One block
    a multiprocessor is resident; a short portion late in a long context fills few of them, and each walks the whole
    context, so its keys are split until the blocks about cover the device."""
    group = nq // nkv
    blocks = nkv * sum(-(-n * group // 256) for n in lengths)
    if window < 0:      # chunks of -window positions: a portion's rows see their own chunk, and the chunk's start may be far from theirs
        longest = max(min(s + n, -window + n) for s, n in zip(starts, lengths))
    else:
        longest = max(min(s + n, window + n) if window > 0 else s + n for s, n in zip(starts, lengths))
    tiles = -(-longest // 64)
    if tiles < PREFILL_SPLIT_FROM_TILES:
        return 1
    return int(max(1, min((sms or sm_count()) // max(1, blocks), tiles // PREFILL_TILES_PER_SPLIT, PREFILL_MAX_SPLITS)))


def paged_prefill_tcgen05(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, T, requests, max_q_len, nq, nkv, d,
                          page_size, scale, window, splits=1, sink=False, sigmoid=False, head_bias=None):
    """Prefill attention on tcgen05 tensor cores: 128 (query, head) rows a block, head sizes 64 and 128.
    ``splits`` > 1 shares the keys of each pair of row tiles out over that many blocks and merges their results."""
    out = torch.empty((T, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    part = scratch(k_cache.device, 4 * T * nq * splits * (d + 1)) if splits > 1 else None
    _run(_bf16(), "fe_paged_prefill_tcgen05", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(max_q_len), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _c_int(_attention_mode(sink, sigmoid)), _c_int(splits), _ptr(part),
         _c_ll(T), _ptr(status_word(k_cache.device)), _ptr(head_bias), _stream())
    return out


def paged_attention(qkv, k_cache, v_cache, block_table, ctx, nq, nkv, d, page_size, scale, window, upcoming=None, sink=False,
                    weights="softmax", head_bias=None):
    """Causal grouped-query attention of the step's tokens over their requests' pages.
    qkv [T, >= nq d] holds the (rotated) queries in its first nq d columns; returns [T, nq d].
    ``window``: what a query sees of the earlier keys: 0 all of them, w > 0 the last w, -c < 0 those of its own chunk of
    c positions (counted from position 0).  ``sink``: 1 is added to the softmax's denominator.
    ``weights`` "sigmoid": no softmax; a visible key weighs sigmoid(score + head_bias[head]) (``head_bias`` float32 [nq] or
    None), not normalised over the keys.
    float32 runs on CUDA cores (true 32-bit); bfloat16 on tensor cores: the split-KV decode
    kernel when every request brings one token, else a prefill kernel (tcgen05 for portions of
    head size 64 or 128, mma.sync otherwise)."""
    _need_cuda(qkv, k_cache, v_cache, block_table)
    T = qkv.shape[0]
    if qkv.dtype != k_cache.dtype:
        raise TypeError("queries and cache differ in dtype")
    if weights not in ("softmax", "sigmoid") or (weights == "sigmoid" and sink):
        raise ValueError("paged_attention: weights are 'softmax' (with or without a sink) or 'sigmoid'")
    sigmoid = weights == "sigmoid"
    if head_bias is not None:
        _need_cuda(head_bias)
        if not sigmoid or head_bias.dtype != torch.float32 or head_bias.numel() != nq:
            raise ValueError("paged_attention: a head bias goes with sigmoid weights and is float32 [heads]")
    if qkv.dtype == torch.float32 or d > 256:          # the tensor-core kernels take head sizes up to 256
        return paged_attention_simt(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start,
                                    ctx.token_request, T, nq, nkv, d, page_size, scale, window, sink, sigmoid, head_bias)
    requests = ctx.cu_q.numel() - 1
    if ctx.max_q_len == 1 and nq // nkv <= 16:
        # a window or a chunk bounds the keys a token walks (plus the tile of 32 that its first key lies in)
        span = ctx.max_ctx_len if window == 0 else min(ctx.max_ctx_len, abs(window) + 31)
        splits = decode_splits(requests, nkv, span)
        clustered = decode_cluster_splits(splits, span, requests * nkv,
                                          lambda s: clusters_resident(requests, nq, nkv, d, s))
        if clustered:
            return paged_decode_cluster(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, requests,
                                        nq, nkv, d, page_size, scale, window, clustered, sink=sink, sigmoid=sigmoid, head_bias=head_bias)
        return paged_decode_mma(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, requests,
                                nq, nkv, d, page_size, scale, window, splits, upcoming=upcoming, sink=sink, sigmoid=sigmoid,
                                head_bias=head_bias)
    lengths = getattr(ctx, "host_lengths", None)
    if tcgen05_attention_ok(ctx.max_q_len, nq, nkv, d, lengths, getattr(ctx, "host_starts", None)):
        splits = prefill_splits(lengths, ctx.host_starts, nq, nkv, window) if lengths else 1
        return paged_prefill_tcgen05(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, T, requests,
                                     ctx.max_q_len, nq, nkv, d, page_size, scale, window, splits, sink=sink, sigmoid=sigmoid,
                                     head_bias=head_bias)
    return paged_prefill_mma(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, T, requests,
                             ctx.max_q_len, nq, nkv, d, page_size, scale, window, sink=sink, sigmoid=sigmoid, head_bias=head_bias)


# ---- several residual streams, token shift, gated attention, minGRU ---------------------------------------------
FUSES_TOKEN_SHIFT = True        # stream_rmsnorm(..., shift=) does the token shift of a decode step's rows in the same kernel


def stream_rmsnorm(streams, read, weight, eps, out_dtype, update=None, rows=None, shift=None):
    """RMSNorm of u = sum_s read[s] x_s over the residual streams x [S, T, H] (float32; ``read`` None: the plain sum).
    ``update`` (an object with y, gate [T, H] in the compute dtype, gate_bias [H], mix [S, S], write [S]) is put into the
    streams first, in the same kernel: x_t <- sum_s mix[s, t] x_s + write[t] * y * sigmoid(gate + gate_bias), every stream
    from the old ones.  rows=None: all rows, the streams updated in place; rows given: only those rows are read and
    nothing is written back.  ``shift`` = (mu [H], kept [seats, H] float32, state_slots): a step in which row i is request i's
    one token; the token shift of the normed rows is then done in the same kernel and (rows, shifted rows) come back."""
    _need_cuda(streams, read, weight, rows)
    if streams.dim() != 3 or streams.dtype != torch.float32 or not streams.is_contiguous() or weight.dtype != torch.float32:
        raise TypeError("stream_rmsnorm: the residual streams are contiguous float32 [S, T, H], norm weights float32")
    S, T, H = streams.shape
    if read is not None and (read.dtype != torch.float32 or read.numel() != S):
        raise ValueError("stream_rmsnorm: read is float32 [S]")
    y = gate = gate_bias = mix = write = None
    if update is not None:
        y, gate, gate_bias, mix, write = update.y, update.gate, update.gate_bias, update.mix, update.write
        _need_cuda(y, gate, gate_bias, mix, write)
        if y.dtype != out_dtype or gate.dtype != out_dtype or tuple(y.shape) != (T, H) or tuple(gate.shape) != (T, H) \
                or not (y.is_contiguous() and gate.is_contiguous()) or gate_bias.dtype != torch.float32 or gate_bias.numel() != H \
                or mix.dtype != torch.float32 or tuple(mix.shape) != (S, S) or write.dtype != torch.float32 or write.numel() != S \
                or not mix.is_contiguous():
            raise ValueError("stream_rmsnorm: the update's rows are contiguous [T, H] in the compute dtype; bias [H], mix [S, S] and "
                             "write [S] float32")
    n_out = T if rows is None else rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=streams.device)
    mu = kept = seats = shifted = None
    if shift is not None:
        mu, kept, seats = shift
        _need_cuda(mu, kept, seats)
        if rows is not None or mu.dtype != torch.float32 or mu.numel() != H or kept.dtype != torch.float32 or kept.stride(-1) != 1 \
                or kept.shape[-1] < H or seats.numel() != T:
            raise ValueError("stream_rmsnorm: the token shift takes all rows of a step of one token a request; mu float32 [H], kept float32 [seats, H]")
        shifted = torch.empty((T, H), dtype=out_dtype, device=streams.device)
    _run(_core(), "fe_stream_rmsnorm", _ptr(streams), _c_int(S), _c_int(T), _c_int(H), _ptr(read), _ptr(weight), _c_float(eps), _ptr(y),
         _ptr(gate), _ptr(gate_bias), _ptr(mix), _ptr(write), _ptr(rows), _c_int(n_out), _ptr(out), _ptr(mu), _ptr(kept),
         _c_ll(kept.stride(0) if kept is not None else 0), _ptr(seats), _c_int(kept.shape[0] if kept is not None else 0), _ptr(shifted),
         _c_int(_code(out_dtype)), _stream())
    return out if shift is None else (out, shifted)


def token_shift(h, mu, kept, state_slots, cu_q, token_request):
    """h + (h' - h) * mu, h' the row of the token before; a portion's first token takes the row its seat kept (``kept``
    [seats, H] float32, zeros for a seat below 0), which then becomes this step's last row."""
    _need_cuda(h, mu, kept, state_slots, cu_q, token_request)
    T, H = h.shape
    if mu.dtype != torch.float32 or mu.numel() != H or kept.dtype != torch.float32 or kept.stride(-1) != 1 or kept.shape[-1] < H \
            or not h.is_contiguous():
        raise ValueError("token_shift: mu is float32 [H]; the kept rows are float32 with unit stride")
    out = torch.empty_like(h)
    _run(_core(), "fe_token_shift", _ptr(h), _ptr(mu), _ptr(kept), _c_ll(kept.stride(0)), _ptr(state_slots), _ptr(cu_q),
         _ptr(token_request), _ptr(out), _c_int(T), _c_int(H), _c_int(kept.shape[0]), _c_int(_code(h.dtype)), _stream())
    return out


def qkv_conv_rope_norm_cache(projected, conv, history, taps, state_slots, cu_q, token_request, positions, inv_freq, rot_dims,
                             qk_norm, eps, slot_mapping, k_cache, v_cache, heads, kv_heads, dim, vdim, head, page_size,
                             q_weight=None, k_weight=None, temp=None):
    """What attention does between its projection and its scores, in one kernel (csrc/hyper_ops.cu).  ``projected``
    [T, >= channels] holds q | k | v (``heads`` and ``kv_heads`` heads of ``dim``, ``kv_heads`` of ``vdim``).  A causal
    convolution of ``taps`` taps over time per channel (``conv`` [taps, channels] float32, tap by tap, None for none; ``history``
    [seats, (taps - 1) channels] float32 holds every request's last taps - 1 projected rows and is brought up to date), the
    first ``rot_dims`` entries of every query and key head turned by position * inv_freq (pairs i, i + rot_dims/2), queries
    and keys divided by their root mean square (``qk_norm``), keys and values into their cache slots
    [pages, kv_heads, page_size, head] (slot_mapping None: no write) and the queries returned [T, heads head], all padded
    with zeros from dim or vdim to ``head``.  ``q_weight``, ``k_weight`` (float32 [dim]): weights of the query and the key
    norm, shared by the heads.  ``temp`` = (coef, every): the query at position p is then multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1)."""
    _need_cuda(projected, conv, history, state_slots, cu_q, token_request, positions, inv_freq, slot_mapping, k_cache, v_cache,
               q_weight, k_weight)
    if (q_weight is None) != (k_weight is None) or any(w is not None and (w.dtype != torch.float32 or w.numel() != dim)
                                                       for w in (q_weight, k_weight)):
        raise ValueError("qkv_conv_rope_norm_cache: the norm weights are two float32 vectors of the head's query/key size")
    temp_coef, temp_every = (float(temp[0]), int(temp[1])) if temp is not None else (0.0, 1)
    T = projected.shape[0]
    channels = (heads + kv_heads) * dim + kv_heads * vdim
    if projected.dim() != 2 or projected.shape[1] < channels or projected.stride(1) != 1:
        raise ValueError("qkv_conv_rope_norm_cache: projected is [T, >= channels] with unit column stride")
    if k_cache.dtype != projected.dtype or tuple(k_cache.shape[1:]) != (kv_heads, page_size, head) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or v_cache.shape != k_cache.shape:
        raise ValueError("qkv_conv_rope_norm_cache: caches are contiguous [pages, kv_heads, page_size, head] in the compute dtype")
    if conv is not None and (conv.dtype != torch.float32 or tuple(conv.shape) != (taps, channels) or not conv.is_contiguous()):
        raise ValueError("qkv_conv_rope_norm_cache: conv is contiguous float32 [taps, channels]")
    if conv is None:
        taps = 0
    if taps > 1 and (history is None or history.dtype != torch.float32 or history.stride(-1) != 1
                     or history.shape[-1] < (taps - 1) * channels):
        raise ValueError("qkv_conv_rope_norm_cache: history is float32 [seats, (taps - 1) channels]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise ValueError("inv_freq must be float32 [rot_dims / 2]")
    queries = torch.empty((T, heads * head), dtype=projected.dtype, device=projected.device)
    seats = history.shape[0] if history is not None else 0
    _run(_core(), "fe_qkv_conv_rope_norm_cache", _ptr(projected), _c_ll(projected.stride(0)), _ptr(conv), _ptr(history if taps > 1 else None),
         _c_ll(history.stride(0) if history is not None else 0), _c_int(taps), _ptr(state_slots), _ptr(cu_q), _ptr(token_request),
         _ptr(positions), _ptr(inv_freq), _c_int(rot_dims if inv_freq is not None else 0), _c_int(1 if qk_norm else 0), _c_float(eps),
         _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _ptr(queries), _c_int(T), _c_int(heads), _c_int(kv_heads), _c_int(dim),
         _c_int(vdim), _c_int(head), _c_int(page_size), _c_ll(k_cache.shape[0] * page_size), _c_int(seats),
         _c_int(_code(projected.dtype)), _ptr(status_word(projected.device)), _ptr(q_weight), _ptr(k_weight), _c_float(temp_coef),
         _c_int(temp_every), _stream())
    return queries


ROTATION_PAIRS = {"halves": 0, "interleaved": 1}


def qkv_norm_rope_cache(projected, q_weight, k_weight, eps, positions, inv_freq, rot_dims, pairs, value_inv_freq, slot_mapping,
                        k_cache, v_cache, heads, kv_heads, dim, vdim, head, page_size):
    """What attention does between its projection and its scores, second form (csrc/hyper_ops.cu).  ``projected``
    [T, >= channels] holds q | k | v.  One RMS norm over the WHOLE query projection with ``q_weight`` (float32
    [heads dim]) and one over the whole key projection with ``k_weight`` ([kv_heads dim]; both None: no norm), then the
    first ``rot_dims`` entries of every query and key head turned by position * inv_freq, ``pairs`` "interleaved"
    (2i with 2i + 1) or "halves" (i with i + rot_dims/2); the values turned over all ``vdim`` entries by position *
    value_inv_freq (None: as they are); keys and values into their cache slots (slot_mapping None: no write) and the
    queries returned [T, heads head], all padded with zeros to ``head``."""
    _need_cuda(projected, q_weight, k_weight, positions, inv_freq, value_inv_freq, slot_mapping, k_cache, v_cache)
    T = projected.shape[0]
    channels = (heads + kv_heads) * dim + kv_heads * vdim
    if projected.dim() != 2 or projected.shape[1] < channels or projected.stride(1) != 1:
        raise ValueError("qkv_norm_rope_cache: projected is [T, >= channels] with unit column stride")
    if (q_weight is None) != (k_weight is None) or (q_weight is not None and (
            q_weight.dtype != torch.float32 or k_weight.dtype != torch.float32 or q_weight.numel() != heads * dim
            or k_weight.numel() != kv_heads * dim)):
        raise ValueError("qkv_norm_rope_cache: the norm weights are float32 [heads dim] and [kv_heads dim]")
    if k_cache.dtype != projected.dtype or tuple(k_cache.shape[1:]) != (kv_heads, page_size, head) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or v_cache.shape != k_cache.shape:
        raise ValueError("qkv_norm_rope_cache: caches are contiguous [pages, kv_heads, page_size, head] in the compute dtype")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise ValueError("inv_freq must be float32 [rot_dims / 2]")
    if value_inv_freq is not None and (value_inv_freq.dtype != torch.float32 or value_inv_freq.numel() != vdim // 2 or vdim % 2):
        raise ValueError("value_inv_freq must be float32 [vdim / 2]")
    if pairs not in ROTATION_PAIRS:
        raise ValueError(f"unknown layout of rotation pairs {pairs!r}; known: {sorted(ROTATION_PAIRS)}")
    queries = torch.empty((T, heads * head), dtype=projected.dtype, device=projected.device)
    _run(_core(), "fe_qkv_norm_rope_cache", _ptr(projected), _c_ll(projected.stride(0)), _ptr(q_weight), _ptr(k_weight), _c_float(eps),
         _ptr(positions), _ptr(inv_freq), _c_int(rot_dims if inv_freq is not None else 0), _c_int(ROTATION_PAIRS[pairs]),
         _ptr(value_inv_freq), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _ptr(queries), _c_int(T), _c_int(heads), _c_int(kv_heads),
         _c_int(dim), _c_int(vdim), _c_int(head), _c_int(page_size), _c_ll(k_cache.shape[0] * page_size), _c_int(_code(projected.dtype)),
         _ptr(status_word(projected.device)), _stream())
    return queries


def unrotate_heads(mixed, positions, inv_freq, heads, head, vdim, pairs, scale=1.0, out=None):
    """[T, heads vdim]: the first ``vdim`` entries of every head of ``mixed`` [T, heads head] turned BACK by the token's
    position (pair m by -position * inv_freq[m]; ``pairs`` as in ``qkv_norm_rope_cache``), times ``scale``.  ``out``: where
    the rows go (a view with any row stride)."""
    _need_cuda(mixed, positions, inv_freq, out)
    T = mixed.shape[0]
    if tuple(mixed.shape) != (T, heads * head) or not mixed.is_contiguous() or inv_freq.dtype != torch.float32 \
            or inv_freq.numel() != vdim // 2 or vdim % 2 or pairs not in ROTATION_PAIRS:
        raise ValueError("unrotate_heads: mixed is contiguous [T, heads head]; inv_freq float32 [vdim / 2]")
    if out is None:
        out = torch.empty((T, heads * vdim), dtype=mixed.dtype, device=mixed.device)
    elif tuple(out.shape) != (T, heads * vdim) or out.dtype != mixed.dtype or out.stride(1) != 1:
        raise ValueError("unrotate_heads: out is [T, heads vdim] in the compute dtype with unit column stride")
    _run(_core(), "fe_unrotate_heads", _ptr(mixed), _ptr(positions), _ptr(inv_freq), _ptr(out), _c_ll(out.stride(0)), _c_int(T),
         _c_int(heads), _c_int(head), _c_int(vdim), _c_int(ROTATION_PAIRS[pairs]), _c_float(scale), _c_int(_code(mixed.dtype)), _stream())
    return out


def head_gate(mixed, projected, offset, heads, head, vdim, per_element=False, scale=1.0, out=None):
    """[T, heads vdim]: out[t, h, :vdim] = mixed[t, h, :vdim] * sigmoid(projected[t, offset + h]) * scale; ``mixed``
    [T, heads head].  With ``per_element`` the gate of entry j of head h is projected[t, offset + h vdim + j].  ``out``: where
    the rows go (a view with any row stride, for rows that are written side by side with another mixer's)."""
    _need_cuda(mixed, projected, out)
    T = mixed.shape[0]
    gates_needed = heads * vdim if per_element else heads
    if tuple(mixed.shape) != (T, heads * head) or not mixed.is_contiguous() or projected.dtype != mixed.dtype \
            or projected.stride(1) != 1 or projected.shape[1] < offset + gates_needed:
        raise ValueError("head_gate: shapes or dtypes do not fit")
    if out is None:
        out = torch.empty((T, heads * vdim), dtype=mixed.dtype, device=mixed.device)
    elif tuple(out.shape) != (T, heads * vdim) or out.dtype != mixed.dtype or out.stride(1) != 1:
        raise ValueError("head_gate: out is [T, heads vdim] in the compute dtype with unit column stride")
    gates = projected[:, offset:]
    _run(_core(), "fe_head_gate", _ptr(mixed), _ptr(gates), _c_ll(projected.stride(0)), _ptr(out), _c_ll(out.stride(0)), _c_int(T),
         _c_int(heads), _c_int(head), _c_int(vdim), _c_int(1 if per_element else 0), _c_float(scale), _c_int(_code(mixed.dtype)), _stream())
    return out


MINGRU_SPAN = 32              # tokens a block of the blocked recurrence walks; a block then folds up to T / 32 blocks before it,
MINGRU_SPAN_LONG = 64         # so portions from 4,096 tokens on take blocks of 64
MINGRU_BLOCKED_FROM = 256     # portions at least this long are scanned in blocks


def mingru_scan(zxg, bias, state, state_slots, cu_q, width, out_dtype, max_q_len=0):
    """The minGRU recurrence over the step's tokens (csrc/hyper_ops.cu): zxg [T, 3 width] float32 holds the projections of
    the gate, the candidate and the output gate; z = sigmoid(. + bias[:W]), u = . + bias[W:], c = u + 1/2 where u >= 0 else
    sigmoid(u), S <- (1 - z) S + z c from state[seat] (float32 [seats, W]; zeros and nothing kept for a seat below 0),
    out = S * silu(g) in ``out_dtype``.  ``max_q_len``: the longest portion of the step; long ones are scanned in blocks."""
    _need_cuda(zxg, bias, state, state_slots, cu_q)
    T, W = zxg.shape[0], int(width)
    if zxg.dtype != torch.float32 or tuple(zxg.shape) != (T, 3 * W) or not zxg.is_contiguous() or bias.dtype != torch.float32 \
            or bias.numel() != 2 * W or state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[-1] < W:
        raise ValueError("mingru_scan: zxg is contiguous float32 [T, 3 W], bias float32 [2 W], the state float32 [seats, W]")
    requests = cu_q.numel() - 1
    out = torch.empty((T, W), dtype=out_dtype, device=zxg.device)
    span, folds = 0, None
    if max_q_len >= MINGRU_BLOCKED_FROM:
        span = MINGRU_SPAN if max_q_len < 4096 else MINGRU_SPAN_LONG
        need = _core().fe_mingru_scan_scratch_floats(_c_int(requests), _c_int(W), _c_int(max_q_len), _c_int(span))
        folds = torch.empty(max(int(need), 1), dtype=torch.float32, device=zxg.device)
    _run(_core(), "fe_mingru_scan", _ptr(zxg), _ptr(bias), _ptr(state), _c_ll(state.stride(0)), _ptr(state_slots), _ptr(cu_q), _ptr(out),
         _c_int(requests), _c_int(W), _c_int(state.shape[0]), _c_int(max_q_len), _c_int(span), _ptr(folds), _c_int(_code(out_dtype)),
         _stream())
    return out


# ---- the stream: hashed pair embedding, grouped norm, average over depth, activations ---------------------------
def embedding_hashed_pairs(token_ids, table, pair_table, previous, state_slots, cu_q, q_start, token_request,
                           buckets, mul_prev, mul_cur):
    """float32 rows [T, H] = table[token] + pair_table[(previous token * mul_prev + token * mul_cur) mod buckets], the
    table's last row (``buckets``) at position 0.  ``previous`` (int32 [seats, 1]) holds every seat's last token of the
    step before and is brought up to date; a seat below 0 keeps nothing."""
    _need_cuda(token_ids, table, pair_table, previous, state_slots, cu_q, q_start, token_request)
    T, (V, H) = token_ids.numel(), table.shape
    if previous.dtype != torch.int32 or not previous.is_contiguous() or pair_table.dtype != table.dtype \
            or tuple(pair_table.shape) != (buckets + 1, H):
        raise ValueError("embedding_hashed_pairs: previous is int32 [seats, 1]; the pair table is [buckets + 1, H] in the table's dtype")
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _run(_core(), "fe_embedding_hashed_pairs", _ptr(token_ids), _ptr(table), _ptr(pair_table), _ptr(previous), _ptr(state_slots),
         _ptr(cu_q), _ptr(q_start), _ptr(token_request), _ptr(out), _c_int(T), _c_int(H), _c_int(V), _c_int(buckets),
         _c_ll(mul_prev), _c_ll(mul_cur), _c_int(previous.shape[0]), _c_int(_code(table.dtype)),
         _ptr(status_word(table.device)), _stream())
    return out


def add_group_rmsnorm(residual, delta, weight, eps, groups, out_dtype, rows=None):
    """Fused residual add + RMSNorm in ``groups`` equal consecutive parts of a row, each with its own root mean square;
    ``rows`` as in ``add_rmsnorm``."""
    _need_cuda(residual, delta, weight, rows)
    T, H = residual.shape
    if residual.dtype != torch.float32 or weight.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream and norm weights are float32")
    if delta is not None and (delta.dtype != out_dtype or delta.shape != residual.shape or not delta.is_contiguous()):
        raise ValueError("add_group_rmsnorm: delta must be contiguous, shaped like the residual, in the compute dtype")
    n_out = T if rows is None else rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
    _run(_core(), "fe_add_group_rmsnorm", _ptr(residual), _ptr(delta), _ptr(weight), _c_float(eps), _ptr(out), _ptr(rows),
         _c_int(n_out), _c_int(H), _c_int(groups), _c_int(T), _c_int(_code(out_dtype)), _stream())
    return out


def depth_average(history, x, mixed, fed, alpha, depth):
    """history[depth + 1] = x + (mixed + fed); x <- sum_j alpha[j] history[j] over j = 0 .. depth + 1, in place, float32.
    history [layers + 1, T, H] float32 (entry 0 is set to x first when depth is 0); ``fed`` may be None."""
    _need_cuda(history, x, mixed, fed, alpha)
    if history.dtype != torch.float32 or x.dtype != torch.float32 or alpha.dtype != torch.float32 or not x.is_contiguous() \
            or not history.is_contiguous() or tuple(history.shape[1:]) != tuple(x.shape) or history.shape[0] < depth + 2 \
            or alpha.numel() < depth + 2:
        raise ValueError("depth_average: float32 stream [T, H], history [>= depth + 2, T, H], at least depth + 2 weights")
    for branch in (mixed, fed):
        if branch is not None and (branch.shape != x.shape or not branch.is_contiguous() or branch.dtype != mixed.dtype):
            raise ValueError("depth_average: the branches are contiguous, shaped like the stream, of one dtype")
    _run(_core(), "fe_depth_average", _ptr(history), _ptr(x), _ptr(mixed), _ptr(fed), _ptr(alpha), _c_int(depth),
         _c_ll(x.numel()), _c_int(_code(mixed.dtype)), _stream())


ACTIVATIONS = {"tanh": 0, "xielu": 1, "relu2": 2}


def activation(x, kind, params=None):
    """Elementwise, float arithmetic, the input's dtype out: "tanh", "relu2" (the square of relu), or "xielu" with
    params = (p, q) on the device: z > 0: softplus(p) z^2 + z/2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    _need_cuda(x, params)
    if kind not in ACTIVATIONS:
        raise ValueError(f"unknown activation {kind!r}; known: {sorted(ACTIVATIONS)}")
    if not x.is_contiguous() or (params is not None and (params.dtype != torch.float32 or params.numel() < 2)):
        raise ValueError("activation: a contiguous tensor; parameters are two float32 numbers")
    out = torch.empty_like(x)
    _run(_core(), "fe_activation", _ptr(x), _ptr(out), _c_ll(x.numel()), _c_int(ACTIVATIONS[kind]), _ptr(params),
         _c_int(_code(x.dtype)), _stream())
    return out


def linear_activated(x, w, kind):
    """act(x w^T) for an activation without parameters ("relu2", "tanh").  The square of relu is an epilogue of the
    weight-streaming kernel (a handful of rows) and of the tcgen05 kernel (a prompt's worth); otherwise the product, then the
    activation kernel."""
    if kind == "relu2" and not isinstance(x, Prenormed):
        if _fits(x, w) == "skinny":
            return skinny_gemm(x, w, EPI_RELU2)
        if tcgen05_ok(x, w):
            return gemm_tcgen05(x, w, EPI_RELU2)
    return activation(linear(x, w), kind)


# ---- the linear-recurrent mixer ---------------------------------------------------------------------------------
def token_shift_blend(h, mu, state, offset, state_slots, cu_q, token_request):
    """The five blends h + (h' - h) * mu_s of every token with the row before it; a portion's first token takes the row
    its seat kept (``state[seat, offset : offset + H]``, float32), which then becomes this step's last row.  Returns
    ([4, T, H] in h's dtype, [T, H] float32): the blends of the four projections and of the decay."""
    _need_cuda(h, mu, state, state_slots, cu_q, token_request)
    T, H = h.shape
    if mu.dtype != torch.float32 or mu.numel() != 5 * H or state.dtype != torch.float32 or state.stride(1) != 1 or not h.is_contiguous():
        raise ValueError("token_shift_blend: mu is float32 [5 H]; the state rows are float32 with unit stride")
    blends = torch.empty((4, T, H), dtype=h.dtype, device=h.device)
    blend_w = torch.empty((T, H), dtype=torch.float32, device=h.device)
    _run(_core(), "fe_token_shift_blend", _ptr(h), _ptr(mu), _ptr(state), _c_ll(state.stride(0)), _c_ll(offset), _ptr(state_slots),
         _ptr(cu_q), _ptr(token_request), _ptr(blends), _ptr(blend_w), _c_int(T), _c_int(H), _c_int(state.shape[0]),
         _c_int(_code(h.dtype)), _stream())
    return blends, blend_w


def wkv_recurrence(r, k, v, decay_logits, w0, u, state, state_slots, cu_q, heads, dim):
    """out_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T with w_t = exp(-exp(decay_logits_t + w0)),
    per request and head; S [dim, dim] float32 lives in ``state[seat, : heads dim dim]`` from step to step.  r, k, v
    [T, heads dim] in the compute dtype; returns float32 [T, heads dim]."""
    _need_cuda(r, k, v, decay_logits, w0, u, state, state_slots, cu_q)
    T, inner = r.shape
    if inner != heads * dim or decay_logits.dtype != torch.float32 or w0.dtype != torch.float32 or u.dtype != torch.float32 \
            or state.dtype != torch.float32 or state.stride(1) != 1 or k.dtype != r.dtype or v.dtype != r.dtype \
            or not (r.is_contiguous() and k.is_contiguous() and v.is_contiguous() and decay_logits.is_contiguous()):
        raise ValueError("wkv_recurrence: r, k, v contiguous [T, heads dim] of one dtype; decay, w0, u and the state float32")
    out = torch.empty((T, inner), dtype=torch.float32, device=r.device)
    _run(_core(), "fe_wkv_recurrence", _ptr(r), _ptr(k), _ptr(v), _ptr(decay_logits), _ptr(w0), _ptr(u), _ptr(state),
         _c_ll(state.stride(0)), _ptr(state_slots), _ptr(cu_q), _ptr(out), _c_int(cu_q.numel() - 1), _c_int(heads), _c_int(dim),
         _c_int(state.shape[0]), _c_int(_code(r.dtype)), _stream())
    return out


def head_rmsnorm_gate(out, weight, g, eps, heads, out_dtype, scale=1.0, into=None):
    """Every head of ``out`` (float32 [T, heads dim]) divided by its root mean square, times ``weight`` (None: a unit norm),
    times silu(g), times ``scale``.  ``g`` and ``into`` (where the rows go) may be views with any row stride."""
    _need_cuda(out, weight, g, into)
    T, inner = out.shape
    if out.dtype != torch.float32 or (weight is not None and weight.dtype != torch.float32) or g.dtype != out_dtype \
            or tuple(g.shape) != (T, inner) or not out.is_contiguous() or g.stride(1) != 1 or inner % heads:
        raise ValueError("head_rmsnorm_gate: float32 rows and weight, a gate of the same shape in the compute dtype")
    y = into if into is not None else torch.empty((T, inner), dtype=out_dtype, device=out.device)
    if tuple(y.shape) != (T, inner) or y.dtype != out_dtype or y.stride(1) != 1:
        raise ValueError("head_rmsnorm_gate: the rows go to [T, heads dim] in the compute dtype with unit column stride")
    _run(_core(), "fe_head_rmsnorm_gate", _ptr(out), _ptr(weight), _ptr(g), _c_ll(g.stride(0)), _ptr(y), _c_ll(y.stride(0)),
         _c_float(eps), _c_float(scale), _c_int(T), _c_int(heads), _c_int(inner // heads), _c_int(_code(out_dtype)), _stream())
    return y


# ---- retention -----------------------------------------------------------------------------------------------------
def rotate_heads(projected, heads, dim, positions, inv_freq, rot_dims, scales):
    """float32 [T, heads dim]: the first ``heads * dim`` columns of ``projected`` (any row stride) as heads of ``dim``, the
    first ``rot_dims`` entries of each turned by position * inv_freq (pairs i, i + rot_dims/2); ``scales``
    ((count, factor), (count, factor)) multiplies the first run of heads by one factor and the rest by another."""
    _need_cuda(projected, positions, inv_freq)
    T = projected.shape[0]
    if projected.dim() != 2 or projected.shape[1] < heads * dim or projected.stride(1) != 1:
        raise ValueError("rotate_heads: projected is [T, >= heads dim] with unit column stride")
    scales = tuple(scales)
    if not 1 <= len(scales) <= 2 or sum(count for count, _ in scales) != heads:
        raise ValueError("rotate_heads: one or two runs of heads that together are all of them")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise ValueError("inv_freq must be float32 [rot_dims / 2]")
    out = torch.empty((T, heads * dim), dtype=torch.float32, device=projected.device)
    _run(_core(), "fe_rotate_heads", _ptr(projected), _c_ll(projected.stride(0)), _ptr(positions), _ptr(inv_freq),
         _c_int(rot_dims if inv_freq is not None else 0), _ptr(out), _c_int(T), _c_int(heads), _c_int(dim), _c_int(scales[0][0]),
         _c_float(scales[0][1]), _c_float(scales[-1][1]), _c_int(_code(projected.dtype)), _stream())
    return out


# a step whose longest portion has this many tokens or more runs the recurrence in blocks of tokens
RETENTION_CHUNKS_FROM = 32


def retention_scan(qk, values, decay, state, state_slots, cu_q, heads, dim, vdim, max_q_len=0):
    """S <- decay_h S + k_t v_t^T, o_t = S^T q_t per request and head over the step's tokens (csrc/retention.cu); S [dim, vdim]
    float32 lives in ``state[seat, : heads dim vdim]`` (zeros and nothing kept for a seat below 0).  qk float32
    [T, 2 heads dim] (queries, then keys); values [T, heads vdim] with any row stride; returns float32 [T, heads vdim]."""
    _need_cuda(qk, values, decay, state, state_slots, cu_q)
    T = qk.shape[0]
    if qk.dtype != torch.float32 or tuple(qk.shape) != (T, 2 * heads * dim) or not qk.is_contiguous() or decay.dtype != torch.float32 \
            or decay.numel() != heads or state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[-1] < heads * dim * vdim \
            or tuple(values.shape) != (T, heads * vdim) or values.stride(1) != 1:
        raise ValueError("retention_scan: qk is contiguous float32 [T, 2 heads dim], values [T, heads vdim], decay float32 [heads], "
                         "the state float32 [seats, >= heads dim vdim]")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=qk.device)
    if max_q_len >= RETENTION_CHUNKS_FROM:
        # long portions: blocks of tokens summed side by side and chained (three launches) instead of a walk token by token
        block = _core().fe_retention_chunk_tokens()
        sums = torch.empty((T // block + cu_q.numel() - 1, heads * dim * vdim), dtype=torch.float32, device=qk.device)
        _run(_core(), "fe_retention_chunks", _ptr(qk), _ptr(values), _c_ll(values.stride(0)), _ptr(decay), _ptr(state),
             _c_ll(state.stride(0)), _ptr(state_slots), _ptr(cu_q), _ptr(out), _ptr(sums), _c_int(cu_q.numel() - 1), _c_int(max_q_len),
             _c_int(heads), _c_int(dim), _c_int(vdim), _c_int(state.shape[0]), _c_int(_code(values.dtype)), _stream())
        return out
    _run(_core(), "fe_retention_scan", _ptr(qk), _ptr(values), _c_ll(values.stride(0)), _ptr(decay), _ptr(state), _c_ll(state.stride(0)),
         _ptr(state_slots), _ptr(cu_q), _ptr(out), _c_int(cu_q.numel() - 1), _c_int(heads), _c_int(dim), _c_int(vdim),
         _c_int(state.shape[0]), _c_int(_code(values.dtype)), _stream())
    return out


def retention_decode(projected, heads, dim, vdim, positions, inv_freq, rot_dims, key_scale, decay, state, state_slots, eps, out_dtype,
                     scale=1.0, into=None):
    """A step of ONE token a request in one kernel (csrc/retention.cu): ``projected`` [R, >= 2 heads dim + 2 heads vdim] =
    q | k | v | g (any row stride); rotation of q and k, the keys times ``key_scale``, S <- decay_h S + k v^T in
    ``state[seat]`` (zeros and nothing kept for a seat below 0), o = S^T q, every head of o divided by its root mean square,
    times silu(g), times ``scale``.  Returns [R, heads vdim] in ``out_dtype`` (``into`` where given, a view with any row stride)."""
    _need_cuda(projected, positions, inv_freq, decay, state, state_slots, into)
    R = projected.shape[0]
    inner = heads * vdim
    if projected.dim() != 2 or projected.shape[1] < 2 * heads * dim + 2 * inner or projected.stride(1) != 1 or projected.dtype != out_dtype \
            or decay.dtype != torch.float32 or decay.numel() != heads or state.dtype != torch.float32 or state.stride(-1) != 1 \
            or state.shape[-1] < heads * dim * vdim or state_slots.numel() < R or positions.numel() < R:
        raise ValueError("retention_decode: projected [R, q | k | v | g] in the compute dtype, decay float32 [heads], the state float32 "
                         "[seats, >= heads dim vdim], a seat and a position per row")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise ValueError("inv_freq must be float32 [rot_dims / 2]")
    y = into if into is not None else torch.empty((R, inner), dtype=out_dtype, device=projected.device)
    if tuple(y.shape) != (R, inner) or y.dtype != out_dtype or y.stride(1) != 1:
        raise ValueError("retention_decode: the rows go to [R, heads vdim] in the compute dtype with unit column stride")
    _run(_core(), "fe_retention_decode", _ptr(projected), _c_ll(projected.stride(0)), _ptr(positions), _ptr(inv_freq),
         _c_int(rot_dims if inv_freq is not None else 0), _c_float(key_scale), _ptr(decay), _ptr(state), _c_ll(state.stride(0)),
         _ptr(state_slots), _ptr(y), _c_ll(y.stride(0)), _c_float(eps), _c_float(scale), _c_int(R), _c_int(heads), _c_int(dim),
         _c_int(vdim), _c_int(state.shape[0]), _c_int(_code(out_dtype)), _stream())
    return y


# ---- attention over a cached latent ------------------------------------------------------------------------------
def batched_linear(x, w, token_major=False):
    """x [B, M, K] (a view with any row and batch strides, unit stride along K) times w [B, N, K]^T, one small matrix a
    batch entry (a head).  Returns [B, M, N], or [M, B N] with ``token_major``.  float32 runs the true 32-bit product
    on CUDA cores; bfloat16 the library's batched product with float accumulation."""
    _need_cuda(x, w)
    B, M, K = x.shape
    N = w.shape[1]
    if w.shape[0] != B or w.shape[2] != K or x.stride(2) != 1 or w.stride(2) != 1 or x.dtype != w.dtype:
        raise ValueError(f"batched_linear: shapes {tuple(x.shape)} x {tuple(w.shape)}")
    if x.dtype == torch.float32:
        if token_major:
            out = torch.empty((M, B * N), dtype=torch.float32, device=x.device)
            ldc, sc = B * N, N
        else:
            out = torch.empty((B, M, N), dtype=torch.float32, device=x.device)
            ldc, sc = N, M * N
        _run(_core(), "fe_gemm_fp32_batched", _ptr(x), _c_ll(x.stride(1)), _c_ll(x.stride(0)), _ptr(w), _c_ll(w.stride(1)),
             _c_ll(w.stride(0)), _ptr(out), _c_ll(ldc), _c_ll(sc), _c_int(M), _c_int(N), _c_int(K), _c_int(B), _stream())
        return out
    y = torch.bmm(x, w.transpose(1, 2))
    return y.transpose(0, 1).reshape(M, B * N) if token_major else y


def latent_prepare(q, q_latent, down, norm_weight, eps, positions, inv_freq, rot_dims, slot_mapping, rows,
                   heads, dim, rot_dim, rank, row, page_size):
    """What a step of attention over a cached latent does around the attention kernel (csrc/latent.cu): the latent
    through its RMS norm, the shared key part and the heads' query parts rotated (interleaved pairs of the first
    ``rot_dims`` entries, float32 angles), this step's rows [latent | key part | 0] into their cache slots
    (``rows`` [pages, 1, page_size, row]; slot_mapping None: no write), and the queries [T, heads row] =
    [q_latent | rotated query part | 0] per head.  q [T, heads (dim + rot_dim)], q_latent [heads, T, rank] in the
    compute dtype; down [T, rank + rot_dim] float32, or None for a layer that reads the rows another layer cached: only
    the queries are made then."""
    _need_cuda(q, q_latent, down, norm_weight, positions, inv_freq, slot_mapping, rows)
    T = q.shape[0]
    if inv_freq.dtype != torch.float32 or tuple(q.shape) != (T, heads * (dim + rot_dim)) or tuple(q_latent.shape) != (heads, T, rank) \
            or inv_freq.numel() != rot_dims // 2 or not (q.is_contiguous() and q_latent.is_contiguous()):
        raise ValueError("latent_prepare: shapes or dtypes do not fit")
    if down is not None and (down.dtype != torch.float32 or norm_weight is None or norm_weight.dtype != torch.float32
                             or tuple(down.shape) != (T, rank + rot_dim) or not down.is_contiguous()):
        raise ValueError("latent_prepare: the latent's projection is contiguous float32 [T, rank + rot_dim], its norm weight float32")
    if down is None:
        slot_mapping = None
    if rows.dtype != q.dtype or tuple(rows.shape[1:]) != (1, page_size, row) or not rows.is_contiguous():
        raise ValueError("latent_prepare: the cache is contiguous [pages, 1, page_size, row] in the compute dtype")
    queries = torch.empty((T, heads * row), dtype=q.dtype, device=q.device)
    _run(_core(), "fe_latent_prepare", _ptr(q), _ptr(q_latent), _ptr(down), _ptr(norm_weight), _c_float(eps), _ptr(positions),
         _ptr(inv_freq), _c_int(rot_dims), _ptr(slot_mapping), _ptr(rows), _c_ll(rows.shape[0] * page_size), _ptr(queries),
         _c_int(T), _c_int(heads), _c_int(dim), _c_int(rot_dim), _c_int(rank), _c_int(row), _c_int(_code(q.dtype)),
         _ptr(status_word(q.device)), _stream())
    return queries


# ---- a routed feed-forward ---------------------------------------------------------------------------------------
def route_top(logits, top, scale, over_chosen=False, correction=None, groups=(1, 1)):
    """(int32 [T, top], float32 [T, top]): per token the ``top`` largest softmax scores over all experts (float32, ties
    to the lower index) times ``scale``, and their experts.  ``over_chosen``: the ``top`` largest logits are chosen and the
    weights are the softmax over those alone (times ``scale``).  ``correction`` (float32, a number per expert) is added to
    the scores for the choice only.  ``groups`` = (count, keep): the experts form ``count`` equal groups of neighbours, a
    group's score is its largest (corrected) score, and only experts of the ``keep`` best groups can be chosen."""
    _need_cuda(logits, correction)
    T, experts = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise TypeError("route_top: router logits are contiguous float32")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != experts):
        raise ValueError("route_top: the correction is float32, a number per expert")
    count, keep = (int(g) for g in groups)
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _run(_core(), "fe_route_top", _ptr(logits), _ptr(chosen), _ptr(weights), _c_int(T), _c_int(experts), _c_int(top),
         _c_float(scale), _c_int(1 if over_chosen else 0), _ptr(correction), _c_int(count), _c_int(keep), _stream())
    return chosen, weights


ROUTED_TCGEN05_MIN_PAIRS = 1024     # fewer sorted rows than this: the mma.sync tiles of the core library
ROUTED_TCGEN05_MIN_K = 1024          # narrower experts: level or behind (512 x 384: 0.090 against 0.052 ms at 2,048 rows)


ROUTED_SINGLE = ("relu2",)            # activations of experts without a gate: one matrix up, one down


def routed_tcgen05_ok(h, pairs, H, F) -> bool:
    """Whether the two products of a routed feed-forward run on the grouped tcgen05 GEMM: bfloat16, a prompt's worth of
    rows, widths whose rows start on 16-byte boundaries."""
    return (h.dtype == torch.bfloat16 and pairs >= ROUTED_TCGEN05_MIN_PAIRS and H % 8 == 0 and F % 8 == 0
            and min(H, F) >= ROUTED_TCGEN05_MIN_K and h.data_ptr() % 16 == 0)


def _routed_experts_tcgen05(h, chosen, weights, gate_up, down, shared, limit=0.0, single=False, identity=0):
    """The routed feed-forward with its products on tcgen05 tensor cores: plan (counting sort, row tiles of 128 per
    expert), the rows of h gathered into sorted order, gate/up with the activation in the epilogue, down into float32,
    combination.  Everything stays on the device."""
    T, H = h.shape
    experts, F2, _ = gate_up.shape
    F, top = (F2 if single else F2 // 2), chosen.shape[1]
    pairs = T * top
    most_tiles = -(-pairs // 128) + experts
    dev = h.device
    plan = torch.empty(experts + 1 + 2 * pairs + 4 + 2 * most_tiles, dtype=torch.int32, device=dev)
    offsets, rest = plan[:experts + 1], plan[experts + 1:]
    row_of_pair, pair_of_row, rest = rest[:pairs], rest[pairs:2 * pairs], rest[2 * pairs:]
    tiles, tile_expert, tile_row0 = rest[:4], rest[4:4 + most_tiles], rest[4 + most_tiles:4 + 2 * most_tiles]
    status = status_word(dev)
    core, tensor = _core(), _bf16()
    _run(core, "fe_routed_plan", _ptr(chosen), _c_int(pairs), _c_int(experts), _c_int(128), _ptr(offsets), _ptr(row_of_pair),
         _ptr(pair_of_row), _ptr(tiles), _ptr(tile_expert), _ptr(tile_row0), _ptr(status), _c_int(identity), _stream())
    rows = torch.empty((pairs, H), dtype=torch.bfloat16, device=dev)
    _run(core, "fe_routed_gather", _ptr(h), _ptr(pair_of_row), _c_int(top), _ptr(rows), _c_int(pairs), _c_ll(H * 2),
         _ptr(offsets[experts:]), _stream())
    act = torch.empty((pairs, F), dtype=torch.bfloat16, device=dev)
    _run(tensor, "fe_gemm_tcgen05_grouped", _ptr(rows), _ptr(gate_up), _ptr(act), _c_int(pairs), _c_int(experts), _c_int(F if single else 2 * F),
         _c_int(H), _c_int(EPI_RELU2 if single else EPI_SWIGLU), _ptr(tiles), _ptr(tile_expert), _ptr(tile_row0), _ptr(offsets), _c_float(limit), _ptr(status), _stream())
    y = torch.empty((pairs, H), dtype=torch.float32, device=dev)
    _run(tensor, "fe_gemm_tcgen05_grouped", _ptr(act), _ptr(down), _ptr(y), _c_int(pairs), _c_int(experts), _c_int(H), _c_int(F),
         _c_int(EPI_F32), _ptr(tiles), _ptr(tile_expert), _ptr(tile_row0), _ptr(offsets), _c_float(0.0), _ptr(status), _stream())
    out = torch.empty((T, H), dtype=h.dtype, device=dev)
    _run(core, "fe_routed_combine", _ptr(y), _ptr(row_of_pair), _ptr(weights), _ptr(shared), _ptr(out), _c_int(T), _c_int(top),
         _c_int(H), _c_int(_code(h.dtype)), _ptr(h) if identity else None, _stream())
    return out


def routed_experts(h, chosen, weights, gate_up, down, shared=None, activation="silu", limit=0.0, identity=0):
    """out[t] = sum_c weights[t, c] * down_e( silu(gate_e h_t) * up_e h_t ) with e = chosen[t, c], plus ``shared`` [T, H] if
    given; gate_up [experts, 2F, H] ([gate; up] per expert), down [experts, H, F].  ``activation`` "clamped": with
    g = min(gate_e h_t, limit) and u = clamp(up_e h_t, -limit, limit) an expert is down_e( g sigmoid(1.702 g) (u + 1) ).
    The (token, choice) pairs are sorted by expert on the device and every expert multiplies its own rows (csrc/routed.cu):
    nothing comes back to the host.  ``activation`` "relu2": experts without a gate; ``gate_up`` is then [experts, F, H] and
    an expert is down_e( relu(up_e h_t)^2 ).  ``identity``: choices in [experts, experts + identity) stand for experts that
    return their input: out[t] += weight * h_t."""
    _need_cuda(h, chosen, weights, gate_up, down, shared)
    T, H = h.shape
    experts, F2, _ = gate_up.shape
    single = activation in ROUTED_SINGLE
    F, top = (F2 if single else F2 // 2), chosen.shape[1]
    if tuple(gate_up.shape) != (experts, F if single else 2 * F, H) or tuple(down.shape) != (experts, H, F) or gate_up.dtype != h.dtype \
            or down.dtype != h.dtype or not (gate_up.is_contiguous() and down.is_contiguous() and h.is_contiguous()) \
            or chosen.dtype != torch.int32 or weights.dtype != torch.float32 \
            or (shared is not None and (shared.dtype != h.dtype or shared.shape != h.shape or not shared.is_contiguous())):
        raise ValueError("routed_experts: shapes or dtypes do not fit")
    if activation not in ("silu", "clamped", "relu2") or (activation == "clamped" and not limit > 0.0):
        raise ValueError("routed_experts: the activation is 'silu', 'relu2' or 'clamped' with a positive limit")
    limit = float(limit) if activation == "clamped" else 0.0
    if routed_tcgen05_ok(h, T * top, H, F):
        return _routed_experts_tcgen05(h, chosen, weights, gate_up, down, shared, limit, single, identity)
    lib = _core()
    need = lib.fe_routed_experts_workspace(_c_int(T), _c_int(top), _c_int(experts), _c_int(H), _c_int(F), _c_int(_code(h.dtype)))
    work = torch.empty(need, dtype=torch.uint8, device=h.device)
    out = torch.empty((T, H), dtype=h.dtype, device=h.device)
    _run(lib, "fe_routed_experts", _ptr(h), _ptr(chosen), _ptr(weights), _ptr(gate_up), _ptr(down), _ptr(shared), _ptr(out),
         _ptr(work), _c_ll(need), _c_int(T), _c_int(top), _c_int(experts), _c_int(H), _c_int(F), _c_int(_code(h.dtype)),
         _c_float(limit), _ptr(status_word(h.device)), _c_int(1 if single else 0), _c_int(identity), _stream())
    return out


def sample(logits, temperature, top_k, seed, draw, blocks: int = 0):
    """int32 [R]: one token per row of float32 logits [R, V]; see csrc/sampling.cu.  ``blocks``: how many thread
    blocks (a cluster of 1, 2, 4 or 8) share a row; 0 lets the kernel library choose by the number of rows.  The
    tokens do not depend on it."""
    _need_cuda(logits, temperature, top_k, seed, draw)
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise TypeError("sample: logits must be float32 with unit column stride")
    if temperature.dtype != torch.float32 or top_k.dtype != torch.int32 or seed.dtype != torch.int64 \
            or draw.dtype != torch.int64:
        raise TypeError("sample: temperature float32, top_k int32, seed and draw int64")
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if blocks:
        _run(_core(), "fe_sample_blocks", _ptr(logits), _c_ll(logits.stride(0)), _c_int(R), _c_int(V), _ptr(temperature),
             _ptr(top_k), _ptr(seed), _ptr(draw), _ptr(out), _c_int(blocks), _stream())
    else:
        _run(_core(), "fe_sample", _ptr(logits), _c_ll(logits.stride(0)), _c_int(R), _c_int(V), _ptr(temperature),
             _ptr(top_k), _ptr(seed), _ptr(draw), _ptr(out), _stream())
    return out


# ---- a whole decoder layer as one call --------------------------------------------------------------------------
import ctypes as _ct


class _FeLayer(_ct.Structure):
    """Mirror of ``struct FeLayer`` (csrc/layer_executor.cu): field for field, in its order."""
    _fields_ = [(n, _ct.c_void_p) for n in ("input_norm", "post_norm", "qkv_weight", "qkv_bias", "out_weight", "gate_up_weight",
                                             "down_weight", "inv_freq")] + \
               [("eps", _ct.c_float), ("scale", _ct.c_float)] + \
               [(n, _ct.c_int) for n in ("hidden", "nq", "nkv", "d", "intermediate", "rot", "window")]


class _FeStep(_ct.Structure):
    """Mirror of ``struct FeStep``."""
    _fields_ = [(n, _ct.c_void_p) for n in ("positions", "slot_mapping", "block_table", "cu_q", "q_start", "residual", "workspace",
                                             "attention_scratch", "status")] + \
               [("workspace_bytes", _ct.c_longlong)] + \
               [(n, _ct.c_int) for n in ("T", "R", "bt_stride", "max_q_len", "page_size", "num_pages", "attention", "splits",
                                         "gate_up_tcgen05")]


NATIVE_LAYER_MIN_ROWS = SKINNY_MAX_ROWS + 1      # fewer rows take the fused weight-streaming kernels, one by one
_workspace: dict = {}
_native_off = False           # set when cuBLAS could not be found from the library: kernel by kernel from then on


class NativeLayer:
    """The weights and sizes of one pre-norm attention + SwiGLU layer in the form ``fe_layer_forward`` takes them (the
    cache is the step's: a model may be run over one cache manager after another).  Holds references to the tensors
    it points at."""

    def __init__(self, input_norm, post_norm, eps, qkv_weight, qkv_bias, out_weight, gate_up_weight, down_weight, inv_freq,
                 rot, nq, nkv, d, scale, window):
        self.keep = (input_norm, post_norm, qkv_weight, qkv_bias, out_weight, gate_up_weight, down_weight, inv_freq)
        _need_cuda(*[t for t in self.keep if t is not None])
        self.hidden, self.intermediate = int(out_weight.shape[0]), int(down_weight.shape[1])
        self.nq, self.nkv, self.d, self.window = nq, nkv, d, window
        self.c = _FeLayer(_ptr(input_norm), _ptr(post_norm), _ptr(qkv_weight), _ptr(qkv_bias), _ptr(out_weight),
                          _ptr(gate_up_weight), _ptr(down_weight), _ptr(inv_freq),
                          float(eps), float(scale), self.hidden, nq, nkv, d, self.intermediate, int(rot), int(window))

    @staticmethod
    def fits(*matrices) -> bool:
        return all(m is not None and m.is_cuda and m.dtype == torch.bfloat16 and m.is_contiguous() and m.data_ptr() % 16 == 0
                   and m.shape[1] % 8 == 0 for m in matrices)


def _layer_workspace(device, nbytes: int) -> torch.Tensor:
    have = _workspace.get(device)
    if have is None or have.numel() < nbytes:
        with torch.inference_mode(False):
            have = _workspace[device] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return have


def native_step(ctx, group, layer: NativeLayer, residual, write_cache: bool):
    """The step's side of ``fe_layer_forward`` for layers of this shape: built once per step and cache group."""
    T, requests = residual.shape[0], ctx.cu_q.numel() - 1
    nq, nkv, d = layer.nq, layer.nkv, layer.d
    scratch_bytes = 0
    if ctx.max_q_len == 1 and nq // nkv <= 16:
        splits = decode_splits(requests, nkv, ctx.max_ctx_len)
        clustered = decode_cluster_splits(splits, ctx.max_ctx_len, requests * nkv,
                                          lambda s: clusters_resident(requests, nq, nkv, d, s))
        kind, splits = (0, clustered) if clustered else (1, splits)
        if kind == 1:
            scratch_bytes = _bf16().fe_paged_decode_scratch_bytes(_c_int(requests), _c_int(nq), _c_int(d), _c_int(splits))
    elif tcgen05_attention_ok(ctx.max_q_len, nq, nkv, d, ctx.host_lengths, ctx.host_starts):
        kind, splits = 2, prefill_splits(ctx.host_lengths, ctx.host_starts, nq, nkv, layer.window)
        scratch_bytes = 4 * T * nq * splits * (d + 1) if splits > 1 else 0
    else:
        kind, splits = 3, 1
    need = _bf16().fe_layer_workspace_bytes(_c_int(T), _c_int(layer.hidden), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(layer.intermediate))
    work = _layer_workspace(residual.device, need)
    attention_scratch = scratch(residual.device, scratch_bytes) if scratch_bytes else None
    gate_up_tcgen05 = T >= TCGEN05_MIN_ROWS and layer.hidden >= TCGEN05_MIN_K
    step = _FeStep(_ptr(ctx.positions), _ptr(group.slot_mapping) if write_cache else None, _ptr(group.block_table), _ptr(ctx.cu_q),
                   _ptr(ctx.q_start), _ptr(residual), _ptr(work), _ptr(attention_scratch), _ptr(status_word(residual.device)),
                   work.numel(), T, requests, int(group.block_table.shape[1]), int(ctx.max_q_len), int(group.page_size),
                   int(group.storage.shape[2]), kind, int(splits), 1 if gate_up_tcgen05 else 0)
    step.keep = (work, attention_scratch, residual)
    # entry points of this package behind one layer, counted as ``_run`` counts them: two norms, rotation and cache
    # write, attention (with its merge, if any), the activation or the fused gate/up product
    step.launches = 5
    return step


def layer_forward(layer: NativeLayer, step, k_cache, v_cache, pending, out):
    """One layer through ``fe_layer_forward``; False when the library cannot (no cuBLAS in the process): the caller
    then runs the layer kernel by kernel, now and from then on."""
    global _native_off, launches
    lib = _bf16()
    rc = lib.fe_layer_forward(_ct.byref(layer.c), _ct.byref(step), _ptr(k_cache), _ptr(v_cache), _ptr(pending), _ptr(out), _stream())
    if rc == 3:
        _native_off = True
        return False
    if rc != 0:
        raise RuntimeError(f"fe_layer_forward failed: {lib.fe_last_error().decode()}")
    launches += step.launches
    return True


def native_layers_usable(ctx) -> bool:
    return (not _native_off and ctx.dtype == torch.bfloat16 and ctx.num_tokens >= NATIVE_LAYER_MIN_ROWS
            and not torch.cuda.is_current_stream_capturing())
