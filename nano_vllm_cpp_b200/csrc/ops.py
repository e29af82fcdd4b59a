"""ctypes binding of the CUDA library: one Python function per launcher.

Every function takes torch CUDA tensors, checks what the kernel assumes (dtype, contiguity,
sizes), launches on torch's current stream and raises ``KernelError`` on a refusal or a
CUDA error.  There is no CPU fallback: on a machine without the library (and without nvcc to
build it) importing the ops fails with the reason.
"""
from __future__ import annotations

import ctypes
import os
import re

import torch

from . import build as _build


# The launchers' prototypes are read from the sources (every ``NV_API`` function of csrc/*.cu) and given to ctypes,
# which then converts plain Python numbers and addresses itself and refuses a call with the wrong number of arguments.
_C_TYPES = {"int": ctypes.c_int, "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
            "float": ctypes.c_float, "double": ctypes.c_double, "void": None, "cudaStream_t": ctypes.c_void_p,
            "const char*": ctypes.c_char_p}


def _c_type(text: str):
    text = " ".join(text.replace("*", " * ").split())
    if "*" in text:
        return ctypes.c_char_p if text.replace("const ", "").startswith("char") else ctypes.c_void_p
    text = text.replace("const ", "")
    try:
        return _C_TYPES[text]
    except KeyError:
        raise KernelError(f"cannot read the C type {text!r} of a launcher's prototype") from None


def _declare(lib: ctypes.CDLL) -> None:
    """Sets ``argtypes`` and ``restype`` of every exported launcher from its definition in the sources."""
    proto = re.compile(r"NV_API\s+([\w\s\*]+?)\s*\b(nv_\w+)\s*\(([^)]*)\)\s*\{", re.S)
    for name in sorted(os.listdir(_build.CSRC)):
        if not name.endswith(".cu"):
            continue
        with open(os.path.join(_build.CSRC, name)) as f:
            text = f.read()
        for ret, fn, args in proto.findall(text):
            types = []
            for a in (x.strip() for x in args.split(",")):
                if not a or a == "void":
                    continue
                m = re.match(r"(.*?)(\w+)$", a, re.S)              # the type is what stands before the name
                types.append(_c_type(m.group(1)))
            f_ = getattr(lib, fn)
            f_.argtypes = types
            f_.restype = _c_type(ret)

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}
_ERR = {-2: "unsupported dtype", -3: "bad size", -4: "size not supported by this kernel",
        -5: "kernel set-up failed"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA library {path}: {e}") from None
        _declare(_lib)
        _lib.nv_set_dependent_launch(_early())
    return _lib


_launches = 0


def launch_count() -> int:
    """How many launcher calls have been made so far (each launches this library's kernels)."""
    return _launches


def add_launches(n: int) -> None:
    """Launches replayed from a CUDA graph, counted at its capture."""
    global _launches
    _launches += n


class KernelTimes:
    """CUDA-event timers per kernel class, off unless asked for:

        with ops.KernelTimes() as kt:
            runner.step(...)
        rows = kt.summary()        # [{"name", "calls", "ms", "flops", "bytes"}], largest first

    While it is active every launcher call records an event behind its launch; the time between two consecutive
    events of a stream is booked to the later launch (so a gap before a kernel counts as its own).  Steps must run
    outside CUDA graphs to be seen.  ``flops`` and ``bytes`` are what the launcher knows from its arguments (matrix
    sizes); 0 where it knows nothing."""

    def __init__(self):
        self.records = []           # (name, start event, end event, flops, bytes)
        self.last = {}

    def __enter__(self):
        global _timer
        torch.cuda.synchronize()
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        self.last = {}
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None
        torch.cuda.synchronize()

    def mark(self) -> None:
        """The next launch's time starts here (the model calls this when a step's kernels begin, so that the host's
        preparation of the step is not booked to its first kernel)."""
        stream = torch.cuda.current_stream()
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        self.last[stream.cuda_stream] = e

    def note(self, name: str, flops: float, nbytes: float) -> None:
        stream = torch.cuda.current_stream()
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        self.records.append((name, self.last.get(stream.cuda_stream, self.start), e, flops, nbytes))
        self.last[stream.cuda_stream] = e

    def summary(self) -> list:
        torch.cuda.synchronize()
        rows = {}
        for name, a, b, flops, nbytes in self.records:
            r = rows.setdefault(name, {"name": name, "calls": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            r["calls"] += 1
            r["ms"] += a.elapsed_time(b)
            r["flops"] += flops
            r["bytes"] += nbytes
        return sorted(rows.values(), key=lambda r: -r["ms"])


_timer = None


def timing() -> bool:
    """True while a ``KernelTimes`` is active: work that would run on a second stream stays on the first then, so
    that every kernel's time is its own."""
    return _timer is not None


def mark_step() -> None:
    if _timer is not None:
        _timer.mark()


def _check(code: int, what: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    global _launches
    _launches += 1
    if _timer is not None and code == 0:
        _timer.note(what, flops, nbytes)
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        f = lib().nv_error_string
        f.restype = ctypes.c_char_p
        return f(code).decode()
    except Exception:
        return "?"


# torch's own fast accessors of the current device and its current stream (a step makes some four hundred
# launches, and ``torch.cuda.current_stream()`` costs ten microseconds a time); the public call where they are missing
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    """The address of a tensor's first element (None: a null pointer)."""
    return None if t is None else t.data_ptr()


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_contig(*ts) -> None:
    for t in ts:
        if t is None:
            continue
        _need(t.is_cuda, "tensor is not on a CUDA device")
        _need(t.is_contiguous(), "tensor is not contiguous")


def _i32(*ts) -> None:
    for t in ts:
        if t is not None:
            _need(t.dtype == torch.int32, f"index tensor must be int32, found {t.dtype}")


# ----------------------------------------------------------------------------- error flag
class ErrorFlag:
    """A device int that kernels set (to 1 + the offending row) instead of trapping."""

    def __init__(self, device):
        self.t = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self, what: str) -> None:
        v = int(self.t.item())
        if v:
            self.t.zero_()
            if v >= 0x7000:
                raise KernelError(f"{what}: a kernel gave up waiting on a barrier (code {v:#x}); its output is invalid")
            raise KernelError(f"{what}: a kernel reported a bad index at row/pair {v - 1}")


# ----------------------------------------------------------------------------- plain ops
def random_fill(out, key: int, mean: float, std: float) -> None:
    """``out[i] = mean + z_i * std`` with z_i a function of (key, i) alone (see weights/random_values.py, whose
    host function gives the same bits)."""
    _cuda_contig(out)
    _check(lib().nv_random_fill(_p(out), dt(out), out.numel(), ctypes.c_ulonglong(key & (2**64 - 1)),
                                mean, std, _stream()), "random_fill")


def embedding(ids, table, out, err: ErrorFlag, feed=None, copies: int = 1, scale: float = 1.0) -> None:
    """``feed``: int32 tokens that negative ids point into (id ``-(r + 1)`` reads ``feed[r]``).  ``copies``: a row of
    ``out`` [T, copies * H] holds the token's row that many times, side by side.  ``scale`` multiplies the row."""
    _cuda_contig(ids, table, out, feed)
    _i32(ids, feed)
    T, (V, H) = ids.numel(), table.shape
    _need(out.dtype == torch.float32 and out.shape == (T, copies * H), "embedding: out must be float32 [T, copies * H]")
    _check(lib().nv_embedding(_p(ids), _p(feed), _p(table), dt(table), _p(out), T, H, V, copies,
                              float(scale), _p(err.t), _stream()), "embedding")


def add_rmsnorm(x, branch, w, eps: float, out, out32=None, *, mix=None, branch2=None, branch_weight=None,
                branch_eps: float = 0.0) -> None:
    """x (+= branch (+ branch2)); out = rmsnorm(x) * w; optional float32 copy of out.

    ``mix`` = (rows, index, weight, dense, gate_logit) gives the branch as a sum that has not been taken yet:
    ``sigmoid(gate_logit[t]) * dense[t] + sum_r weight[t, r] * rows[index[t, r]]`` (dense and gate_logit may be
    None); it is summed inside the kernel instead of by ``moe_combine`` first.

    ``branch_weight`` (float32 [H]): the branch, in whichever form, passes an RMS norm of its own first,
    ``x += rms(branch) * branch_weight`` with ``branch_eps`` inside its root, in the same pass over the row."""
    _cuda_contig(x, branch, branch2, w, out, out32, branch_weight)
    _need(branch_weight is None or (branch_weight.dtype == torch.float32 and branch_weight.numel() == x.shape[1]
                                    and (branch is not None or mix is not None)),
          "add_rmsnorm: a branch weight is float32 [H] and comes with a branch")
    T, H = x.shape
    _need(x.dtype == torch.float32, "add_rmsnorm: the residual stream is float32")
    _need(branch2 is None or (branch is not None and branch2.dtype == torch.float32 and branch2.shape == x.shape),
          "add_rmsnorm: a second branch comes with a first and is float32 and shaped like x")
    _need(branch is None or (branch.dtype == torch.float32 and branch.shape == x.shape),
          "add_rmsnorm: branch must be float32 and shaped like x")
    _need(w.numel() == H and out.shape == x.shape, "add_rmsnorm: shape mismatch")
    _need(out32 is None or (out32.dtype == torch.float32 and out32.shape == x.shape), "add_rmsnorm: out32")
    rows = index = weight = dense = gate = None
    R, gate_ld = 0, 1
    if mix is not None:
        _need(branch is None, "add_rmsnorm: a branch or a mix, not both")
        rows, index, weight, dense, gate = mix
        _cuda_contig(rows, index, weight, dense)
        R = index.shape[1]
        _need(R <= ADD_RMSNORM_MAX_MIX, f"add_rmsnorm: at most {ADD_RMSNORM_MAX_MIX} rows are mixed per token")
        _need(rows.dtype == torch.float32 and rows.shape[1] == H and weight.dtype == torch.float32
              and index.dtype == torch.int32 and index.shape == (T, R) and weight.shape == (T, R),
              "add_rmsnorm: mix shapes")
        _need(dense is None or (dense.dtype == torch.float32 and dense.shape == x.shape), "add_rmsnorm: mix dense term")
        if gate is not None:
            _need(gate.dtype == torch.float32, "add_rmsnorm: gate logits are float32")
            gate_ld = gate.stride(0) if gate.dim() >= 1 else 1
    if H % 4 == 0:
        for t_ in (x, branch, branch2, out, out32, rows, dense):
            _need(t_ is None or t_.data_ptr() % 16 == 0, "add_rmsnorm: rows must start on 16-byte boundaries")
    _check(lib().nv_add_rmsnorm(_p(x), _p(branch), _p(branch2), _p(w), dt(w), eps, _p(out), dt(out),
                                _p(out32), T, H, _p(rows), _p(index), _p(weight), R, _p(dense),
                                _p(gate), gate_ld, _p(branch_weight), float(branch_eps), _stream()), "add_rmsnorm")


ADD_RMSNORM_MAX_MIX = 64


EPILOGUE_ACTS = {"gelu_erf": 2, "gelu_tanh": 3, "silu": 4, "relu2": 7}
EPILOGUE_XIELU = 5          # given as the tuple ("xielu", p0, p1) with its two positive numbers
EPILOGUE_GLU_CLAMPED = 6    # with ``swiglu``: the tuple ("glu_clamped", limit, slope) makes the pairing of gate and up rows
                            # g = min(g, limit), u = clamp(u, -limit, limit), g sigmoid(slope g) (u + 1)


def _epilogue(swiglu: bool, act) -> int:
    """What the products' launchers take in their ``swiglu`` argument: 0 nothing, 1 the SwiGLU pairing, or the code
    of a unary activation that every output value passes after the bias."""
    if act is None:
        return 1 if swiglu else 0
    if isinstance(act, tuple):
        if swiglu:
            _need(len(act) == 3 and act[0] == "glu_clamped" and act[1] > 0, "a pairing with numbers is ('glu_clamped', limit, slope)")
            return EPILOGUE_GLU_CLAMPED
        _need(len(act) == 3 and act[0] == "xielu", "a product's activation with numbers is ('xielu', p0, p1)")
        return EPILOGUE_XIELU
    _need(not swiglu and act in EPILOGUE_ACTS, f"a product's activation is one of {sorted(EPILOGUE_ACTS)} and excludes swiglu")
    return EPILOGUE_ACTS[act]


def _act_numbers(act):
    """The two numbers that a product's launcher takes beside the activation's code (0, 0 where it has none)."""
    return (float(act[1]), float(act[2])) if isinstance(act, tuple) else (0.0, 0.0)


def gemm_plain(a, w, out, *, bias=None, a_rows=None, swiglu=False, M=None, tiles=None, act=None) -> None:
    """out[m, :] = a[a_rows[m] or m, :] @ w.T (+ bias), or silu(gate) * up with ``swiglu``, or with ``act``
    (gelu_erf, gelu_tanh, silu) that function of every value.

    ``tiles`` = (tile_expert, tile_row0, tile_rows, num_tiles) selects the grouped form, where w is
    [E, rows, K]."""
    _cuda_contig(w, bias, a_rows)
    _need(a.stride(-1) == 1 and out.stride(-1) == 1, "gemm: rows must be dense")
    K = a.shape[1]
    grouped = tiles is not None
    n_rows_w = w.shape[-2]
    _need(w.shape[-1] == K, f"gemm: inner sizes differ ({K} vs {w.shape[-1]})")
    N = n_rows_w // 2 if swiglu else n_rows_w
    _need(not swiglu or n_rows_w % 2 == 0, "gemm: swiglu needs an even number of weight rows")
    if M is None:
        M = a_rows.numel() if a_rows is not None else a.shape[0]
    _need(out.shape[0] >= M and out.shape[1] == N, f"gemm: out is {tuple(out.shape)}, need [{M}, {N}]")
    _i32(a_rows)
    if grouped:
        te, tr0, tr, nt = tiles
        _i32(te, tr0, tr, nt)
        stride = w.stride(0)
        max_tiles = te.numel()
    else:
        te = tr0 = tr = nt = None
        stride = 0
        max_tiles = 0
    if bias is not None:
        _need(bias.numel() == N, "gemm: bias length")
    _check(lib().nv_gemm_plain(_p(a), dt(a), a.stride(0), _p(a_rows),
                               _p(w), dt(w), stride,
                               _p(bias), (dt(bias) if bias is not None else 0),
                               _p(out), dt(out), out.stride(0),
                               M, N, K, _epilogue(swiglu, act),
                               _p(te), _p(tr0), _p(tr), _p(nt), max_tiles, *_act_numbers(act), _stream()), "gemm_plain")


def rowdot(a, w, out, wide: bool = False) -> None:
    """out[t, n] = a[t, :] . w[n, :] for float32 rows and a short matrix (float32 or bfloat16), float32 out.
    ``wide``: the many-rows kernel (another summation order; see small_ops.cu)."""
    _cuda_contig(w)
    _need(a.dtype == torch.float32 and out.dtype == torch.float32 and a.stride(1) == 1 and out.stride(1) == 1,
          "rowdot: float32 rows")
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (T, N), "rowdot: shapes")
    scratch = None
    if wide:        # a long K is cut into ranges whose sums a second kernel adds
        n = int(lib().nv_rowdot_scratch_floats(T, N, K, 1))
        if n:
            scratch = torch.empty(n, dtype=torch.float32, device=a.device)
    _check(lib().nv_rowdot(_p(a), a.stride(0), _p(w), dt(w), _p(out), out.stride(0),
                           T, N, K, (1 if wide else 0), _p(scratch), _stream()), "rowdot")


def attention_decode_usable(k_cache, D: int) -> bool:
    return bool(lib().nv_attention_decode_usable(D, k_cache.shape[2], dt(k_cache)))


def attention_decode(qkv, k_cache, v_cache, block_table, row_entry, positions, scale: float, window: int, out,
                     Hq: int, Hkv: int, D: int, max_context: int, rows=None, err=None, sink_score=None,
                     float_weights: bool = False, softcap: float = 0.0) -> None:
    """One query row per request (``rows``: which batch rows; None = all) against its paged keys.  ``qkv``: rows
    whose first Hq * D elements are the query heads.  ``sink_score``: a further key with that score and no value
    in every softmax.  ``float_weights``: the weights keep all their bits in the product with the values (the
    tensor-core form takes them as three bfloat16 terms instead of one rounded one; the kernel that gives a lane a
    chunk of a key, which other head sizes and a sink go to, multiplies in float32).  ``softcap`` > 0: a scaled score s
    becomes ``softcap * tanh(s / softcap)`` (the lane-per-chunk kernel)."""
    _cuda_contig(qkv, k_cache, v_cache, block_table, row_entry, positions, out, rows)
    _i32(block_table, row_entry, positions, rows)
    R = qkv.shape[0] if rows is None else rows.numel()
    page = k_cache.shape[2]
    L = lib()
    splits = L.nv_attention_decode_splits(R, Hq, Hkv, max_context, num_sms())
    scratch = counts = None
    if splits > 1:
        scratch = torch.empty(R * Hq * splits * (D + 2), dtype=torch.float32, device=qkv.device)
        counts = _split_counts(qkv.device)
    _check(L.nv_attention_decode(_p(qkv), dt(qkv), qkv.shape[1], _p(k_cache), _p(v_cache),
                                 dt(k_cache), _p(block_table), block_table.shape[1], _p(row_entry),
                                 _p(positions), _p(rows), R, scale, window, _p(out),
                                 dt(out), Hq, Hkv, D, page, k_cache.shape[0],
                                 splits, _p(scratch), _p(err.t if err is not None else _global_err().t),
                                 _p(counts), (counts.numel() if counts is not None else 0),
                                 (0 if sink_score is None else 1), float(sink_score or 0.0),
                                 (1 if float_weights else 0), float(softcap), _stream()),
           "attention_decode")


_counts = {}


def _split_counts(device):
    """Zeros that the decode attention kernel counts finished splits in (and sets back to zero itself): one array
    per device, for kernels that run one after the other, as a step's do."""
    key = torch.device(device)
    if key not in _counts:
        _counts[key] = torch.zeros(1 << 16, dtype=torch.int32, device=key)
    return _counts[key]


def attention_prefill_tile_rows() -> int:
    return int(lib().nv_attention_prefill_tile_rows())


def attention_prefill(qkv, k_cache, v_cache, block_table, cu_rows, entry_pos0, max_tiles: int, scale: float,
                      window: int, out, Hq: int, Hkv: int, D: int, err=None, min_rows: int = 1,
                      kernel: str = "auto", sink_score=None, weight_terms: int = 1, softcap: float = 0.0) -> None:
    """bfloat16 rows of any mix of portions against their paged keys: the tcgen05 kernel for head sizes 64 and
    128 and pages of 16, 32 or 64 keys, else the mma.sync kernel (``kernel="mma"`` asks for that one).  Entries
    with fewer than ``min_rows`` rows are skipped and their rows of ``out`` left as they are.
    ``weight_terms`` = 3: the float32 weights enter the product with the values as three bfloat16 terms, all their
    bits (either kernel).  ``sink_score``: a further key with that score and no value in every softmax; ``softcap``
    > 0: a scaled score s becomes ``softcap * tanh(s / softcap)`` before mask and softmax (either kernel)."""
    _cuda_contig(qkv, k_cache, v_cache, block_table, cu_rows, entry_pos0, out)
    _i32(block_table, cu_rows, entry_pos0)
    _need(qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(out.shape == (qkv.shape[0], Hq * D), "attention_prefill: out shape")
    S = entry_pos0.numel()
    L = lib()
    page = k_cache.shape[2]
    _need(kernel in ("auto", "mma"), "attention_prefill: kernel is 'auto' or 'mma'")
    _need(weight_terms in (1, 3), "attention_prefill: the weights are one bfloat16 term or three")
    if kernel == "auto" and L.nv_attention_prefill_tc_usable(D, page):
        _check(L.nv_attention_prefill_tc(_p(qkv), qkv.shape[1], qkv.shape[0], _p(k_cache), _p(v_cache),
                                         k_cache.shape[0], _p(block_table), block_table.shape[1],
                                         _p(cu_rows), _p(entry_pos0), S, max_tiles, scale,
                                         window, _p(out), Hq, Hkv, D, page,
                                         min_rows, weight_terms, _p(err.t if err is not None else _global_err().t),
                                         (0 if sink_score is None else 1), float(sink_score or 0.0), float(softcap),
                                         _stream()),
               "attention_prefill_tc")
        return
    _check(L.nv_attention_prefill(_p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table),
                                  block_table.shape[1], _p(cu_rows), _p(entry_pos0), S,
                                  max_tiles, scale, window, _p(out), Hq, Hkv,
                                  D, page, min_rows, (0 if sink_score is None else 1), float(sink_score or 0.0),
                                  weight_terms, float(softcap), _stream()), "attention_prefill")


def attention_prefill_wide_usable(D: int, key_span: int, Dv: int) -> bool:
    """Whether ``attention_prefill_wide`` takes these sizes: a key length ``key_span * D`` up to 512 and values up to
    256, both multiples of 16."""
    return bool(lib().nv_attention_prefill_wide_usable(D, key_span, Dv))


def attention_prefill_wide_tile_rows() -> int:
    return int(lib().nv_attention_prefill_wide_tile_rows())


def attention_prefill_wide(q, k_cache, v_cache, block_table, cu_rows, entry_pos0, max_tiles: int, scale: float,
                           window: int, out, Hq: int, Hkv: int, D: int, Dv: int, *, keep_first: int = 0, sinks=None,
                           key_span: int = 1, min_rows: int = 1, max_rows: int = 0, narrow: bool = False,
                           heads: bool = False, max_keys: int = 0) -> None:
    """bfloat16 rows of any mix of portions (single rows too) against paged keys of ``D`` and values of ``Dv``
    elements, on the tensor cores with float32 softmax weights (three bfloat16 terms).  ``q`` [T, Hq * key_span * D]:
    with ``key_span`` = Hkv > 1 a query head is scored against all kv heads' keys side by side (queries mixed across
    heads).  ``keep_first``: the first so many positions stay visible behind the window; ``sinks`` [Hq] float32: a
    learned score without key and value in every softmax.  ``out`` [T, Hq * Dv] bfloat16 or float32.  Entries with
    fewer than ``min_rows`` or (``max_rows`` > 0) more than ``max_rows`` rows are skipped and their rows of ``out``
    left as they are.

    ``narrow``: the form for entries of at most ``attention_wide_narrow_rows()`` rows, decoded tokens above all (it
    skips longer entries): all warps of a CTA work on the entry's rows and share out the keys, and when the step has
    too few entries and heads to fill the multiprocessors, several CTAs share out the key tiles of one entry and head
    and a second kernel merges them (``max_keys``: the most keys any such entry reads, which bounds the shares).

    ``heads`` (where ``attention_wide_heads_usable``): the form for entries of exactly one row whose query heads all
    read the same keys: a CTA takes all heads of the row, so the keys are read once for them (it skips every other
    entry)."""
    _cuda_contig(q, k_cache, v_cache, block_table, cu_rows, entry_pos0, out, sinks)
    _i32(block_table, cu_rows, entry_pos0)
    _f32(sinks)
    T = q.shape[0]
    _need(q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attention_prefill_wide: bfloat16 only")
    _need(out.dtype in (torch.bfloat16, torch.float32) and out.shape == (T, Hq * Dv) and q.shape == (T, Hq * key_span * D),
          "attention_prefill_wide: shapes")
    _need(k_cache.shape[1] == Hkv and k_cache.shape[3] == D and v_cache.shape[3] == Dv and key_span in (1, Hkv),
          "attention_prefill_wide: cache shapes")
    _need(sinks is None or sinks.numel() == Hq, "attention_prefill_wide: one sink per head")
    S = entry_pos0.numel()
    splits, parts = 1, None
    narrow = narrow or heads
    if narrow:
        max_tiles = S
        ctas = max(1, S if heads else S * Hq)
        tile = 64 if key_span * D <= 256 else 32
        key_tiles = max(1, (max(1, max_keys) + tile - 1) // tile)
        splits = max(1, min(32, key_tiles, (2 * num_sms() + ctas - 1) // ctas))
        if splits > 1:
            parts = torch.empty(T * Hq * splits * (Dv + 2), dtype=torch.float32, device=q.device)
    _check(lib().nv_attention_prefill_wide(_p(q), _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1],
                                           _p(cu_rows), _p(entry_pos0), S, max_tiles, scale, window,
                                           keep_first, _p(sinks), _p(out), (1 if out.dtype == torch.float32 else 0), Hq,
                                           Hkv, v_cache.shape[1], D, key_span, Dv, k_cache.shape[2], min_rows,
                                           max_rows, (2 if heads else 1 if narrow else 0), splits, _p(parts), _stream()),
           "attention_prefill_wide")


def attention_wide_heads_usable(D: int, key_span: int, Dv: int, Hq: int, Hkv: int, Hv: int) -> bool:
    """Whether the ``heads`` form of ``attention_prefill_wide`` takes these sizes (``key_span`` = Hkv, at most 16 query
    heads, the value heads' tiles fit in shared memory)."""
    return bool(lib().nv_attention_wide_heads_usable(D, key_span, Dv, Hq, Hkv, Hv))


def attention_wide_narrow_rows() -> int:
    """The most rows of an entry that the narrow form of ``attention_prefill_wide`` takes."""
    return 16


def gemm_plain_tile_m() -> int:
    return int(lib().nv_gemm_plain_tile_m())


def rope_store(qkv, positions, inv_freq, rotary_dim: int, k_cache, v_cache, block_table, row_entry,
               Hq: int, Hkv: int, D: int, write_kv: bool, err: ErrorFlag, rot_positions=None, pair_axis=None) -> None:
    """Turns q and k by their positions and writes k and v to their pages.  ``positions`` [T] are the rows' places
    in their sequences (they pick the cache slot, and the angle unless ``rot_positions`` is given).
    ``rot_positions`` [T] or [T, axes] int32: the coordinates that the pairs are turned by instead, and
    ``pair_axis`` [rotary_dim / 2] int32: which coordinate turns which pair (None: the first)."""
    _cuda_contig(qkv, positions, inv_freq, k_cache, v_cache, block_table, row_entry, rot_positions, pair_axis)
    _i32(positions, block_table, row_entry, rot_positions, pair_axis)
    T = qkv.shape[0]
    axes = 0
    if rot_positions is not None:
        axes = 1 if rot_positions.dim() == 1 else rot_positions.shape[1]
        _need(rot_positions.shape[0] == T and axes >= 1, "rope_store: one row of coordinates per row")
    _need(pair_axis is None or (rot_positions is not None and pair_axis.numel() >= rotary_dim // 2),
          "rope_store: pair_axis needs rot_positions and one entry per pair")
    _need(qkv.shape[1] == (Hq + 2 * Hkv) * D, "rope_store: qkv width")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2, "rope_store: inv_freq")
    page = k_cache.shape[2]
    _need(k_cache.shape[1:] == (Hkv, page, D) and v_cache.shape == k_cache.shape, "rope_store: cache shape")
    _check(lib().nv_rope_store(_p(qkv), dt(qkv), _p(positions), _p(rot_positions), axes, _p(pair_axis),
                               _p(inv_freq), rotary_dim,
                               _p(k_cache), _p(v_cache), dt(k_cache), _p(block_table),
                               block_table.shape[1], _p(row_entry), T, Hq, Hkv,
                               D, page, (1 if write_kv else 0), _p(err.t), _stream()),
           "rope_store")


def paged_attention_plain(qkv, k_cache, v_cache, block_table, row_entry, positions, scale: float, window: int,
                          out, Hq: int, Hkv: int, D: int) -> None:
    _cuda_contig(qkv, k_cache, v_cache, block_table, row_entry, positions, out)
    _i32(block_table, row_entry, positions)
    T = qkv.shape[0]
    page = k_cache.shape[2]
    _need(out.shape == (T, Hq * D), "attention: out shape")
    _check(lib().nv_paged_attention_plain(_p(qkv), dt(qkv), qkv.shape[1], _p(k_cache), _p(v_cache),
                                          dt(k_cache), _p(block_table), block_table.shape[1],
                                          _p(row_entry), _p(positions), scale, window, _p(out),
                                          dt(out), T, Hq, Hkv, D, page,
                                          _stream()), "paged_attention_plain")


ROUTE_SCORES = {"softmax": 0, "sigmoid": 1}


def _route_rule(rule, E: int):
    """``rule`` = None (softmax, no bias, weights as they are) or (score kind, choice bias [E] float32 or None,
    weight scale): what the routing kernels take as their last three arguments."""
    if rule is None:
        return 0, None, 1.0
    kind, bias, scale = rule
    _need(kind in ROUTE_SCORES, f"router: the score is one of {sorted(ROUTE_SCORES)}")
    _need(bias is None or (kind == "sigmoid" and bias.is_cuda and bias.dtype == torch.float32 and bias.is_contiguous()
                           and bias.numel() == E), "router: the choice bias is float32 [E], with sigmoid scores")
    return ROUTE_SCORES[kind], bias, float(scale)


def router_topk(logits, K: int, renorm: bool, idx, score, C: int = 0, gate_logit=None, rule=None) -> None:
    """``logits`` may be a column slice of a wider float32 matrix (rows ``stride(0)`` apart).  With ``C`` the
    rows of ``idx``/``score`` are K + C wide: C always-on experts E..E+C-1 weighted sigmoid(gate_logit), or 1
    without gate logits.  ``rule``: see ``_route_rule``."""
    _cuda_contig(idx, score)
    _need(logits.is_cuda and logits.stride(1) == 1, "router: logits rows must be dense")
    T, E = logits.shape
    _need(logits.dtype == torch.float32 and score.dtype == torch.float32, "router: float32 logits and scores")
    _i32(idx)
    _need(idx.shape == (T, K + C) and score.shape == (T, K + C), "router: output shapes")
    _need(gate_logit is None or gate_logit.dtype == torch.float32, "router: gate logits")
    mode, bias, wscale = _route_rule(rule, E)
    _check(lib().nv_router_topk(_p(logits), logits.stride(0), T, E, K,
                                (1 if renorm else 0), _p(idx), _p(score), C, _p(gate_logit),
                                (gate_logit.stride(0) if gate_logit is not None else 0), mode, _p(bias), wscale,
                                _stream()),
           "router_topk")


class TileList:
    """Tiles (expert, first row, rows) over an expert-sorted row list, cut by ``tile_m`` rows."""

    def __init__(self, TK: int, E: int, tile_m: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.tile_m = tile_m
        self.max_tiles = max(1, min(TK, (TK + tile_m - 1) // tile_m + E))
        self.tile_expert = torch.empty(self.max_tiles, **i32)
        self.tile_row0 = torch.empty(self.max_tiles, **i32)
        self.tile_rows = torch.empty(self.max_tiles, **i32)
        self.num_tiles = torch.zeros(1, **i32)

    @property
    def arrays(self):
        return (self.tile_expert, self.tile_row0, self.tile_rows, self.num_tiles)


class MoeAlignment:
    """Device buffers of one expert permutation (sizes fixed by T*K and E): counts and offsets per expert,
    the sorted pairs, and one or two tile lists over them (``tile_m2``: a second list cut by another tile
    size, for a product that prefers it; 0 = none)."""

    def __init__(self, TK: int, E: int, tile_m: int, device, tile_m2: int = 0):
        i32 = dict(dtype=torch.int32, device=device)
        self.TK, self.E = TK, E
        self.primary = TileList(TK, E, tile_m, device)
        self.secondary = TileList(TK, E, tile_m2, device) if tile_m2 and tile_m2 != tile_m else None
        self.counts = torch.empty(E, **i32)
        self.offsets = torch.empty(E + 1, **i32)
        self.sorted_token = torch.empty(max(TK, 1), **i32)
        self.pair_pos = torch.empty(max(TK, 1), **i32)

    # the primary list under the names the kernels' wrappers use
    tile_m = property(lambda self: self.primary.tile_m)
    max_tiles = property(lambda self: self.primary.max_tiles)
    tile_expert = property(lambda self: self.primary.tile_expert)
    tile_row0 = property(lambda self: self.primary.tile_row0)
    tile_rows = property(lambda self: self.primary.tile_rows)
    num_tiles = property(lambda self: self.primary.num_tiles)

    @property
    def tiles(self):
        return self.primary.arrays

    def list_for(self, tile_m: int) -> TileList:
        if self.secondary is not None and self.secondary.tile_m == tile_m:
            return self.secondary
        return self.primary


def moe_align(idx, K: int, al: MoeAlignment, err: ErrorFlag, spread_last: int = 0, static_last: int = 0,
              zero=None) -> None:
    """``spread_last``: the tiles of the last so many experts (ones that every row visits) are spread evenly through
    the tile lists instead of standing at their end.  ``static_last`` instead: those experts' pairs sit in row order
    at the end of the permutation and get no tiles (``StaticTiles`` lists them; they can run before the routing).
    ``zero``: a few int32 that the kernel also sets to 0 (the tile counters of the products that follow it)."""
    _cuda_contig(idx)
    _i32(idx)
    T = idx.numel() // K
    _need(T * K == al.TK, "moe_align: buffers were sized for another batch")
    s2 = al.secondary
    _check(lib().nv_moe_align(_p(idx), T, K, al.E, al.tile_m, _p(al.counts),
                              _p(al.offsets), _p(al.sorted_token), _p(al.pair_pos),
                              _p(al.tile_expert), _p(al.tile_row0), _p(al.tile_rows), _p(al.num_tiles), _p(err.t),
                              (s2.tile_m if s2 else 0), _p(s2.tile_expert if s2 else None), _p(s2.tile_row0 if s2 else None),
                              _p(s2.tile_rows if s2 else None), _p(s2.num_tiles if s2 else None), spread_last,
                              static_last, _p(zero), (zero.numel() if zero is not None else 0), _stream()),
           "moe_align")


def moe_route_small_usable(T: int, E: int, K: int, C: int, H: int) -> bool:
    return bool(lib().nv_moe_route_small_usable(T, E, K, C, H))


def moe_route_small(logits, K: int, renorm: bool, C: int, gate_logit, idx, score, al: "MoeAlignment", err, x=None,
                    static: bool = False, zero=None, rule=None):
    """Top-k, expert permutation and (with ``x``, bfloat16 rows) the expert-sorted copy of x, in one launch.
    Returns the sorted copy or None.  ``static``: the C always-on experts' pairs sit in row order at the end of
    the permutation and get no tiles (``static_tiles`` lists them; they can then run before the routing).
    ``zero``: a few int32 that the kernel also sets to 0 (the tile counters of the products that follow it)."""
    T, E = logits.shape
    KT = K + C
    _need(idx.shape == (T, KT) and score.shape == (T, KT) and al.TK == T * KT and al.E == E + C, "route: sizes")
    _need(al.secondary is None, "route: the one-launch routing builds one tile list")
    xs = None
    H = 8
    if x is not None:
        _need(x.dtype == torch.bfloat16 and x.is_contiguous(), "route: bfloat16 rows")
        H = x.shape[1]
        xs = torch.empty((T * KT, H), dtype=x.dtype, device=x.device)
    mode, bias, wscale = _route_rule(rule, E)
    _check(lib().nv_moe_route_small(_p(logits), logits.stride(0), T, E, K,
                                    (1 if renorm else 0), C, _p(gate_logit),
                                    (gate_logit.stride(0) if gate_logit is not None else 0), _p(idx),
                                    _p(score), al.tile_m, _p(al.counts), _p(al.offsets), _p(al.sorted_token),
                                    _p(al.pair_pos), _p(al.tile_expert), _p(al.tile_row0), _p(al.tile_rows),
                                    _p(al.num_tiles), _p(err.t), _p(x), _p(xs), H, (C if static else 0),
                                    _p(zero), (zero.numel() if zero is not None else 0), mode, _p(bias), wscale,
                                    _stream()), "moe_route_small")
    return xs


class StaticTiles:
    """The tiles of C experts E .. E + C - 1 that each take all T rows, in row order, their segments behind the
    T * K routed pairs: what ``moe_route_small(static=True)`` leaves out of its list."""

    def __init__(self, T: int, K: int, E: int, C: int, device):
        self.tile_m = 16 if T <= 16 else (32 if T <= 32 else (64 if T <= 64 else 128))
        experts, row0, rows = [], [], []
        for c in range(C):
            for r in range(0, T, self.tile_m):
                experts.append(E + c)
                row0.append(T * K + c * T + r)
                rows.append(min(self.tile_m, T - r))
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tiles = len(experts)
        self.tile_expert = torch.tensor(experts, **i32)
        self.tile_row0 = torch.tensor(row0, **i32)
        self.tile_rows = torch.tensor(rows, **i32)
        self.num_tiles = torch.tensor([len(experts)], **i32)
        self.x_rows = (T * K, T)


def moe_combine(y, pair_pos, score, shared, gate_logit, out) -> None:
    """``gate_logit``: [T] or a [T, 1] column slice of a wider float32 matrix."""
    _cuda_contig(y, pair_pos, score, shared, out)
    T, K = score.shape
    gate_ld = 1 if gate_logit is None else (gate_logit.stride(0) if gate_logit.dim() >= 1 else 1)
    H = out.shape[1]
    for t in (y, score, shared, gate_logit, out):
        _need(t is None or t.dtype == torch.float32, "moe_combine: float32 tensors")
    _check(lib().nv_moe_combine(_p(y), _p(pair_pos), _p(score), _p(shared), _p(gate_logit), gate_ld,
                                _p(out), T, K, H, _stream()), "moe_combine")


def silu_mul(gu, out) -> None:
    _cuda_contig(gu, out)
    rows, I2 = gu.shape
    _need(out.shape == (rows, I2 // 2), "silu_mul: out shape")
    _check(lib().nv_silu_mul(_p(gu), dt(gu), _p(out), dt(out), rows, I2 // 2,
                             _stream()), "silu_mul")


def gather_rows(src, rows, dst) -> None:
    _cuda_contig(src, rows, dst)
    _i32(rows)
    _need(src.dtype == dst.dtype and dst.shape == (rows.numel(), src.shape[1]), "gather_rows: shapes")
    _check(lib().nv_gather_rows(_p(src), dt(src), _p(rows), _p(dst), rows.numel(),
                                src.shape[1], _stream()), "gather_rows")


def reset_fresh_state(state, entry_slot, entry_pos0) -> None:
    """Zeroes ``state[slot]`` (``state``: [slots, ...]) for every entry whose first position is 0."""
    _cuda_contig(state, entry_slot, entry_pos0)
    _i32(entry_slot, entry_pos0)
    slots = state.shape[0]
    slot_bytes = (state.numel() // max(slots, 1)) * state.element_size()
    _need(slot_bytes % 4 == 0, "reset_fresh_state: a slot's bytes must be a multiple of four")
    _check(lib().nv_reset_fresh_state(_p(state), slot_bytes, slots, _p(entry_slot), _p(entry_pos0),
                                      entry_slot.numel(), _stream()), "reset_fresh_state")


def sync_block_tables(src, lens, rows, entry_slot, tables, step_tables, S: int) -> None:
    """``tables`` [slots, max_blocks] takes in the rows that travelled with the step (``rows[src[e]]`` for the
    entries with ``src[e]`` >= 0) and ``step_tables[e, :lens[e]]`` becomes entry e's table, for e < S."""
    _cuda_contig(src, lens, rows, entry_slot, tables, step_tables)
    _i32(src, lens, rows, entry_slot, tables, step_tables)
    slots, max_blocks = tables.shape
    _need(step_tables.shape == tables.shape and src.numel() >= S and lens.numel() >= S and entry_slot.numel() >= S,
          "sync_block_tables: shapes")
    _check(lib().nv_sync_block_tables(_p(src), _p(lens), _p(rows), _p(entry_slot), _p(tables), _p(step_tables),
                                      S, max_blocks, slots, _stream()), "sync_block_tables")


def delay(micros: int) -> None:
    """Keeps the current stream busy for about ``micros`` microseconds (at most 200,000); for measurements that
    want a step's launches queued before the GPU starts on them."""
    code = lib().nv_delay(int(micros), _stream())
    if code:
        raise KernelError(f"delay: {_ERR.get(code, code)}")


def sample(logits, temperature, u, out) -> None:
    """One token per row: greedy where temperature <= 0, else inverse-CDF with the given u in [0,1)."""
    _cuda_contig(logits, temperature, u, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and temperature.dtype == torch.float32 and u.dtype == torch.float64,
          "sample: logits/temperature float32, u float64")
    _i32(out)
    _need(temperature.numel() == R and u.numel() == R and out.numel() == R, "sample: one entry per row")
    _check(lib().nv_sample(_p(logits), R, V, _p(temperature), _p(u), _p(out), _stream()), "sample")


def sample_nucleus(logits, params, recent, recent_off, out) -> None:
    """One token per row by nucleus (top-p) sampling with a repetition penalty (include/nanovllm/sampler.hpp:46-88).
    ``params``: float64 [R, 4] = (temperature, top_p, penalty, u) per row; ``recent``: int32 ids whose scores are
    divided by the row's penalty, row r's being ``recent[recent_off[r]:recent_off[r + 1]]``."""
    _cuda_contig(logits, params, recent, recent_off, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and params.dtype == torch.float64 and params.shape == (R, 4),
          "sample_nucleus: logits float32 [R, V], params float64 [R, 4]")
    _i32(recent, recent_off, out)
    _need(recent_off.numel() == R + 1 and out.numel() == R, "sample_nucleus: one entry per row")
    work = torch.empty_like(logits)
    _check(lib().nv_sample_nucleus(_p(logits), _p(work), R, V, _p(params), _p(recent), _p(recent_off),
                                   _p(out), _stream()), "sample_nucleus")


# ----------------------------------------------------------------------------- state mixers and their layer pieces
ACTIVATIONS = {"gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "xielu": 3, "relu2": 4}


def _f32(*ts) -> None:
    for t in ts:
        if t is not None:
            _need(t.dtype == torch.float32, f"tensor must be float32, found {t.dtype}")


def branch_norm_add(x, branches, weight, eps: float, out=None, *, branch_weights=None, mix_scale: float = 1.0,
                    mix=None, next_weight=None, next_eps: float = 0.0, out32=None) -> None:
    """``x += rms(y) * weight`` row by row, and ``out`` (float32 or bfloat16, optional) = the new ``x``.
    ``y`` is the one branch, or with ``branch_weights`` ``mix_scale * sum_b rms(branches[b]) * branch_weights[b]``,
    or with ``mix`` = (rows, index, weight, dense, gate_logit) the sum that has not been taken yet (see
    ``add_rmsnorm``).  ``rms(v) = v / sqrt(mean(v^2) + eps)``.  Without branches only ``out = x`` is written.
    ``next_weight``: ``out`` (and ``out32``, a float32 copy) is instead ``rms(x) * next_weight`` of the stream after
    the sum, with ``next_eps``: the input of the sublayer that follows, from the same launch."""
    branches = list(branches or [])
    bws = list(branch_weights or [])
    _cuda_contig(x, weight, out, *branches, *bws)
    _f32(x, weight, *branches, *bws)
    T, H = x.shape
    _need(len(branches) <= 4 and (not bws or len(bws) == len(branches)), "branch_norm_add: up to four branches, a weight for each or for none")
    _need(len(branches) <= 1 or bws, "branch_norm_add: several branches need their weights")
    _need(not branches or (weight is not None and weight.numel() == H), "branch_norm_add: weight")
    for b in branches:
        _need(b.shape == x.shape, "branch_norm_add: a branch is shaped like x")
    for w in bws:
        _need(w.numel() == H, "branch_norm_add: a branch weight has one entry per column")
    _need(out is None or out.shape == x.shape, "branch_norm_add: out shape")
    b4 = branches + [None] * (4 - len(branches))
    w4 = bws + [None] * (4 - len(bws))
    rows = index = mweight = dense = gate = None
    R, gate_ld = 0, 1
    if mix is not None:
        _need(not branches, "branch_norm_add: branches or a mix, not both")
        rows, index, mweight, dense, gate = mix
        _cuda_contig(rows, index, mweight, dense)
        _f32(rows, mweight, dense, gate)
        _i32(index)
        R = index.shape[1]
        _need(rows.shape[1] == H and index.shape == (T, R) and mweight.shape == (T, R)
              and (dense is None or dense.shape == x.shape) and weight is not None and weight.numel() == H,
              "branch_norm_add: mix shapes")
        if gate is not None:
            gate_ld = gate.stride(0) if gate.dim() >= 1 else 1
    _cuda_contig(next_weight, out32)
    _f32(next_weight, out32)
    _need(next_weight is None or next_weight.numel() == H, "branch_norm_add: next_weight")
    _need(out32 is None or (next_weight is not None and out32.shape == x.shape), "branch_norm_add: out32 comes with next_weight")
    _check(lib().nv_branch_norm_add(_p(x), _p(b4[0]), _p(b4[1]), _p(b4[2]), _p(b4[3]), _p(w4[0]), _p(w4[1]), _p(w4[2]),
                                    _p(w4[3]), len(branches), mix_scale, _p(weight), eps, _p(out),
                                    (dt(out) if out is not None else 0), T, H, _p(rows), _p(index), _p(mweight), R,
                                    _p(dense), _p(gate), gate_ld, _p(next_weight), float(next_eps), _p(out32),
                                    _stream()), "branch_norm_add")


def activation(src, out, kind: str, params=(0.0, 0.0)) -> None:
    """``out = act(src)`` elementwise; ``kind``: gelu_erf, gelu_tanh, silu, or xielu with ``params`` = (a, b), both
    positive: ``a z^2 + z / 2`` for z > 0 and ``b (e^z - 1 - z) + z / 2`` for z <= 0."""
    _cuda_contig(src, out)
    _need(src.shape == out.shape and kind in ACTIVATIONS, "activation: shapes or kind")
    _check(lib().nv_activation(_p(src), dt(src), _p(out), dt(out), src.numel(), ACTIVATIONS[kind], float(params[0]),
                               float(params[1]), _stream()), "activation")


def token_gate(gate, ids, table, col0: int, out, err: ErrorFlag, feed=None) -> None:
    """``out[t, j] = gelu_tanh(gate[t, j]) * table[ids[t], col0 + j]`` (negative ids point into ``feed``)."""
    _cuda_contig(ids, table, out, feed)
    _i32(ids, feed)
    T, d = out.shape
    _need(gate.stride(-1) == 1 and gate.shape[0] == T and gate.shape[1] >= d, "token_gate: gate rows")
    _check(lib().nv_token_gate(_p(gate), dt(gate), gate.stride(0), _p(ids), _p(feed), _p(table), dt(table),
                               table.stride(0), col0, d, table.shape[0], _p(out), dt(out), T, _p(err.t), _stream()),
           "token_gate")


def _slot_stride(state) -> int:
    """Elements between two slots of a per-request state array (a slot's own elements are contiguous)."""
    _need(state.is_cuda and state.dtype == torch.float32, "state arrays are float32 on the device")
    inner = state[0]
    _need(inner.is_contiguous(), "a slot of a state array must be contiguous")
    return state.stride(0)


def conv_silu_norm(src, col0: int, C: int, w, taps: int, batch, state, out, *, unit_heads: int = 0, unit_dim: int = 1,
                   unit_eps: float = 0.0, scaled_heads: int = 0, scale: float = 1.0) -> None:
    """Short causal convolution over time per channel (columns col0..col0+C of ``src``), then silu; the first
    ``unit_heads`` heads of ``unit_dim`` channels become unit vectors (the first ``scaled_heads`` times ``scale``).
    ``state`` [slots, taps - 1, C] holds what came before the rows of this step."""
    _cuda_contig(w, out)
    _f32(w, out)
    T = src.shape[0]
    _need(src.stride(-1) == 1 and out.shape == (T, C) and w.shape == (C, taps), "conv_silu_norm: shapes")
    _check(lib().nv_conv_silu_norm(_p(src), dt(src), src.stride(0), col0, C, _p(w), taps, _p(batch.row_entry),
                                   _p(batch.cu_rows), _p(batch.entry_slot), _p(state), _slot_stride(state),
                                   unit_heads, unit_dim, unit_eps, scaled_heads, scale, _p(out), T, _stream()),
           "conv_silu_norm")


def conv_state_update(src, col0: int, C: int, taps: int, batch, state) -> None:
    """After ``conv_silu_norm``: the last ``taps - 1`` inputs of every entry's channels go to its state."""
    _check(lib().nv_conv_state_update(_p(src), dt(src), src.stride(0), col0, C, taps, _p(batch.cu_rows),
                                      _p(batch.entry_slot), _p(state), _slot_stride(state), batch.S, _stream()),
           "conv_state_update")


def scan_usable(dk: int, dv: int, parts: int = 1) -> bool:
    return bool(lib().nv_scan_usable(dk, dv, parts))


def col_scan_usable(dk: int, dv: int) -> bool:
    """Whether the scans that keep a column of a head's matrix in a thread's registers take these sizes."""
    return bool(lib().nv_col_scan_usable(dk, dv))


def channel_scan_usable(dk: int, dv: int) -> bool:
    """Whether the fast form of the delta rule with channel decays takes these sizes (else the plain scan runs)."""
    return bool(lib().nv_channel_scan_usable(dk, dv))


def mlstm_scan(proj, cols: dict, batch, S, n, m, H: int, dk: int, dv: int, cap: float, eps: float, norm_w, out,
               *, den_eps: float = 1e-6, columns: bool = True) -> None:
    """The matrix memory with exponential gating, row by row per entry, from and to the entries' states.
    ``proj`` float32 [T, P] holds q, k, v, the output gate and the two gate pre-activations at ``cols``
    (keys q, k, v, g, i, f).  ``columns``: the kernel that keeps a column per thread where it takes the sizes
    (keys up to 128 long), else the one that keeps the matrix in shared memory."""
    _cuda_contig(proj, norm_w, out)
    _f32(proj, norm_w)
    _need(norm_w.numel() in (dv, H * dv) and out.shape == (proj.shape[0], H * dv), "mlstm_scan: shapes")
    if columns and col_scan_usable(dk, dv):
        T = proj.shape[0]
        raw = torch.empty((T, H, dv + 2), dtype=torch.float32, device=proj.device)
        gate_buf = torch.empty((T, H, 2), dtype=torch.float32, device=proj.device)
        _check(lib().nv_mlstm_col_scan(_p(proj), proj.stride(0), cols["q"], cols["k"], cols["v"], cols["g"], cols["i"],
                                       cols["f"], _p(batch.cu_rows), _p(batch.entry_slot), _p(S), _slot_stride(S), _p(n),
                                       _slot_stride(n), _p(m), _slot_stride(m), H, dk, dv, cap, float(dk) ** -0.5,
                                       den_eps, eps, _p(norm_w), (1 if norm_w.numel() == H * dv and H > 1 else 0),
                                       _p(raw), _p(gate_buf), _p(out), dt(out), batch.S, T, _stream()), "mlstm_col_scan")
        return
    _check(lib().nv_mlstm_scan(_p(proj), proj.stride(0), cols["q"], cols["k"], cols["v"], cols["g"], cols["i"],
                               cols["f"], _p(batch.cu_rows), _p(batch.entry_slot), _p(S), _slot_stride(S), _p(n),
                               _slot_stride(n), _p(m), _slot_stride(m), H, dk, dv, cap, float(dk) ** -0.5, den_eps,
                               eps, _p(norm_w), (1 if norm_w.numel() == H * dv and H > 1 else 0), _p(out), dt(out),
                               batch.S, _stream()), "mlstm_scan")


def gated_delta_scan(qkv, cols: dict, G: int, proj, pcols: dict, A_log, dt_bias, batch, S, H: int, dk: int, dv: int,
                     eps: float, norm_w, out, *, columns: bool = True, channel_decay=None, gate_src=None,
                     gate: str = "silu") -> None:
    """The gated delta rule, row by row per entry.  ``qkv`` float32 [T, C]: q, k, v after convolution and unit norm
    at ``cols`` (q, k, v); ``proj``: output gate, beta and decay pre-activations at ``pcols`` (g, b, a).
    ``columns`` as in ``mlstm_scan``.  ``channel_decay`` (float32 [T, >= a + H * dk]): the decay has one
    pre-activation per head and key channel, at column ``pcols['a']`` of that matrix, and ``dt_bias`` is [H * dk].
    ``gate_src``: the matrix that holds the output gate's pre-activations at ``pcols['g']`` where it is not ``proj``;
    ``gate``: silu or sigmoid."""
    _cuda_contig(qkv, A_log, dt_bias, norm_w, out)
    _f32(qkv, A_log, dt_bias, norm_w)
    _need(proj.stride(-1) == 1 and norm_w.numel() == dv and out.shape == (qkv.shape[0], H * dv), "gated_delta_scan: shapes")
    _need(gate in ("silu", "sigmoid"), "gated_delta_scan: the output gate is silu or sigmoid")
    if channel_decay is not None or gate_src is not None or gate != "silu":
        dec = channel_decay
        if dec is not None:
            _f32(dec)
            _need(dec.stride(-1) == 1 and dec.shape[0] == qkv.shape[0] and dt_bias.numel() == H * dk
                  and dec.shape[1] >= pcols["a"] + H * dk, "gated_delta_scan: channel decays")
        gs = gate_src if gate_src is not None else proj
        _need(gs.stride(-1) == 1 and gs.shape[0] == qkv.shape[0], "gated_delta_scan: gate rows")
        if columns and col_scan_usable(dk, dv) and dec is not None and channel_scan_usable(dk, dv):
            T = qkv.shape[0]
            raw = torch.empty((T, H, dv), dtype=torch.float32, device=qkv.device)
            gate_buf = torch.empty((T, H, 2), dtype=torch.float32, device=qkv.device)
            decays = torch.empty((T, H * dk), dtype=torch.float32, device=qkv.device)
            _check(lib().nv_channel_delta_scan(_p(qkv), qkv.shape[1], cols["q"], cols["k"], cols["v"], G, _p(proj),
                                               dt(proj), proj.stride(0), pcols["b"], _p(dec), dec.stride(0), pcols["a"],
                                               _p(gs), dt(gs), gs.stride(0), pcols["g"], (1 if gate == "sigmoid" else 0),
                                               _p(A_log), _p(dt_bias), _p(batch.cu_rows), _p(batch.entry_slot), _p(S),
                                               _slot_stride(S), H, dk, dv, eps, _p(norm_w), _p(raw), _p(gate_buf),
                                               _p(decays), _p(out), dt(out), batch.S, T, _stream()), "channel_delta_scan")
            return
        _check(lib().nv_gated_delta_scan(_p(qkv), qkv.shape[1], cols["q"], cols["k"], cols["v"], G, _p(proj), dt(proj),
                                         proj.stride(0), pcols["g"], pcols["b"], (0 if dec is not None else pcols["a"]),
                                         _p(A_log), _p(dt_bias), _p(batch.cu_rows), _p(batch.entry_slot), _p(S),
                                         _slot_stride(S), H, dk, dv, eps, _p(norm_w), _p(out), dt(out), batch.S,
                                         _p(dec), (dec.stride(0) if dec is not None else 0), pcols["a"], _p(gs), dt(gs),
                                         gs.stride(0), (1 if dec is not None else 0), (1 if gate == "sigmoid" else 0),
                                         _stream()), "gated_delta_scan")
        return
    if columns and col_scan_usable(dk, dv):
        T = qkv.shape[0]
        raw = torch.empty((T, H, dv), dtype=torch.float32, device=qkv.device)
        gate_buf = torch.empty((T, H, 2), dtype=torch.float32, device=qkv.device)
        _check(lib().nv_gated_delta_col_scan(_p(qkv), qkv.shape[1], cols["q"], cols["k"], cols["v"], G, _p(proj),
                                             dt(proj), proj.stride(0), pcols["g"], pcols["b"], pcols["a"], _p(A_log),
                                             _p(dt_bias), _p(batch.cu_rows), _p(batch.entry_slot), _p(S),
                                             _slot_stride(S), H, dk, dv, eps, _p(norm_w), _p(raw), _p(gate_buf), _p(out),
                                             dt(out), batch.S, T, _stream()), "gated_delta_col_scan")
        return
    _check(lib().nv_gated_delta_scan(_p(qkv), qkv.shape[1], cols["q"], cols["k"], cols["v"], G, _p(proj), dt(proj),
                                     proj.stride(0), pcols["g"], pcols["b"], pcols["a"], _p(A_log), _p(dt_bias),
                                     _p(batch.cu_rows), _p(batch.entry_slot), _p(S), _slot_stride(S), H, dk, dv, eps,
                                     _p(norm_w), _p(out), dt(out), batch.S, None, 0, 0, None, 0, 0, 0, 0, _stream()),
           "gated_delta_scan")


def qk_prepare_store(src, q0: int, k0: int, v0: int, positions, row_entry, block_table, q_weight, k_weight, eps: float,
                     inv_freq, rot_dim: int, interleaved: bool, amplitude: float, q_out, k_cache, v_cache,
                     Hq: int, Hkv: int, D: int, Dv: int, write_kv: bool, err: ErrorFlag, *, v_inv_freq=None,
                     v_rot_dim: int = 0, rot0: int = 0, k_norm_dim: int = 0, norm_always: bool = False,
                     norm_after: bool = False) -> None:
    """Per row: q and k heads RMS-normed over D (weights may be None), their first ``rot_dim`` elements turned in
    pairs by the row's position, q to ``q_out`` [T, Hq * D], k and v to the row's place in their pages.
    ``Hq`` may be 0 (``q_out`` None: only keys and values are written) and ``v_cache`` None (only keys).
    ``v_rot_dim`` > 0: the first so many elements of every value head are turned too, in pairs
    ``(i, i + v_rot_dim / 2)`` by ``position * v_inv_freq[i]``, before they are stored.
    ``rot0``: the turned elements are ``rot0 .. rot0 + rot_dim - 1`` of a head.  ``k_norm_dim`` > 0: a key head's norm is
    taken over, and applied to, its first so many elements only.  ``norm_always``: heads are normed also where the
    weight is None (the weight is then one).  ``norm_after``: the norm follows the turn instead of preceding it."""
    _cuda_contig(positions, row_entry, block_table, q_weight, k_weight, inv_freq, q_out, k_cache, v_cache, v_inv_freq)
    _i32(positions, row_entry, block_table)
    _f32(q_weight, k_weight, inv_freq, v_inv_freq)
    T = src.shape[0]
    page = k_cache.shape[2]
    QP = q_out.shape[1] // Hq if Hq else D
    KP, VP = k_cache.shape[3], (v_cache.shape[3] if v_cache is not None else Dv)   # a head's elements, padded with zeros
    _need(src.stride(-1) == 1 and (Hq == 0 or q_out.shape == (T, Hq * QP)) and QP >= D, "qk_prepare_store: shapes")
    if not write_kv or Hkv == 0:          # nothing is written: only the queries are prepared
        KP, VP = max(KP, D), max(VP, Dv)
    _need(not write_kv or Hkv == 0 or (k_cache.shape[1:3] == (Hkv, page) and KP >= D and VP >= Dv),
          "qk_prepare_store: cache shapes")
    _need(v_cache is None or not write_kv or (v_cache.shape[1:3] == (Hkv, page) and k_cache.dtype == v_cache.dtype),
          "qk_prepare_store: cache shapes")
    _need(rot_dim == 0 or inv_freq.numel() >= rot_dim // 2, "qk_prepare_store: inv_freq")
    _need(v_rot_dim == 0 or (v_inv_freq is not None and v_inv_freq.numel() >= v_rot_dim // 2), "qk_prepare_store: v_inv_freq")
    _check(lib().nv_qk_prepare_store(_p(src), dt(src), src.stride(0), q0, k0, v0, _p(positions), _p(row_entry),
                                     _p(block_table), block_table.shape[1], _p(q_weight), _p(k_weight), eps,
                                     _p(inv_freq), rot_dim, (1 if interleaved else 0), amplitude, _p(q_out),
                                     (dt(q_out) if q_out is not None else 0),
                                     _p(k_cache), _p(v_cache), dt(k_cache), Hq, Hkv, D, Dv, page,
                                     (1 if write_kv else 0), _p(err.t), T, QP, KP, VP, _p(v_inv_freq), v_rot_dim,
                                     rot0, k_norm_dim, (1 if norm_always else 0) | (2 if norm_after else 0),
                                     _stream()), "qk_prepare_store")


def paged_attention_general(q, k_cache, v_cache, block_table, row_entry, positions, scale: float, window: int, out,
                            Hq: int, Hkv: int, D: int, Dv: int, sink_score=None, *, sinks=None, keep_first: int = 0,
                            key_span: int = 1, value_heads: int | None = None, softcap: float = 0.0) -> None:
    """Causal softmax attention of every row over its request's paged keys; values may be wider or narrower than
    keys; ``sink_score``: a further key with that score and no value in every softmax (None: none), ``sinks``
    (float32 [Hq]): one such score per head; ``keep_first``: with a window, the sequence's first so many positions
    stay visible; ``key_span`` = Hkv: a query row holds Hkv * D elements per head and a score is the sum of its
    parts' products with all kv heads' keys (see ``mix_query_heads``); ``v_cache`` None: the values are read where
    the keys are; ``value_heads``: kv heads of the values where that is not ``Hkv``; ``softcap`` > 0: a scaled score
    s becomes ``softcap * tanh(s / softcap)`` before mask and softmax."""
    if v_cache is None:
        v_cache = k_cache
    Hv = Hkv if value_heads is None else value_heads
    _cuda_contig(q, k_cache, v_cache, block_table, row_entry, positions, out, sinks)
    _i32(block_table, row_entry, positions)
    _f32(sinks)
    T = q.shape[0]
    _need(q.shape == (T, Hq * key_span * D) and out.shape == (T, Hq * Dv), "attention: shapes")
    _need(k_cache.shape[1] == Hkv and k_cache.shape[3] == D and v_cache.shape[1] == Hv and v_cache.shape[3] == Dv
          and k_cache.dtype == v_cache.dtype, "attention: cache shapes")
    _need(sinks is None or sinks.numel() == Hq, "attention: one sink per query head")
    _check(lib().nv_paged_attention_general(_p(q), dt(q), _p(k_cache), _p(v_cache), dt(k_cache), _p(block_table),
                                            block_table.shape[1], _p(row_entry), _p(positions), scale, window,
                                            keep_first, (0 if sink_score is None else 1), float(sink_score or 0.0),
                                            _p(sinks), _p(out), dt(out), T, Hq, Hkv, Hv, D, Dv, key_span,
                                            k_cache.shape[2], float(softcap), _stream()),
           "paged_attention_general")


def mix_query_heads(q, mix, out, H: int, G: int, D: int) -> None:
    """``out[t, h, c * D + d] = sum over the heads g of kv head c of mix[h, g] * q[t, g, d]``: the query rows of
    an attention whose scores are mixed across heads before the softmax (``q`` float32 [T, H * D], ``mix`` float32
    [H, H], ``out`` [T, H * G * D])."""
    _cuda_contig(q, mix, out)
    _f32(q, mix)
    T = q.shape[0]
    _need(q.shape == (T, H * D) and mix.shape == (H, H) and out.shape == (T, H * G * D), "mix_query_heads: shapes")
    _check(lib().nv_mix_query_heads(_p(q), _p(mix), _p(out), dt(out), T, H, G, D, _stream()), "mix_query_heads")


def rotate_heads(x, positions, inv_freq, rot_dim: int, sign: float, out, H: int, D: int) -> None:
    """The first ``rot_dim`` elements of every head of ``x`` [T, H * D] turned in pairs ``(i, i + rot_dim / 2)`` by
    ``sign * position * inv_freq[i]``, written to ``out`` (another tensor, any of the two dtypes)."""
    _cuda_contig(x, positions, inv_freq, out)
    _i32(positions)
    _f32(inv_freq)
    T = x.shape[0]
    _need(x.shape == (T, H * D) and out.shape == x.shape and inv_freq.numel() >= rot_dim // 2
          and x.data_ptr() != out.data_ptr(), "rotate_heads: shapes")
    _check(lib().nv_rotate_heads(_p(x), dt(x), _p(positions), _p(inv_freq), rot_dim, float(sign), _p(out), dt(out),
                                 T, H, D, _stream()), "rotate_heads")


def cols_rmsnorm(src, col0: int, n: int, w, eps: float, out) -> None:
    """``out = rms(src[:, col0:col0 + n]) * w`` for float32 rows, the norm over the ``n`` columns."""
    _cuda_contig(w, out)
    _f32(src, w)
    T = src.shape[0]
    _need(src.stride(-1) == 1 and src.shape[1] >= col0 + n and out.shape == (T, n) and w.numel() == n,
          "cols_rmsnorm: shapes")
    _check(lib().nv_cols_rmsnorm(_p(src), src.stride(0), col0, n, _p(w), eps, _p(out), dt(out), T, _stream()),
           "cols_rmsnorm")


def head_project(x, w, out, H: int, K: int, N: int, gate=None, gate_col: int = 0, gate_each: bool = False) -> None:
    """``out[t, h, :] = x[t, h, :] @ w[h]`` for ``x`` [T, H * K] and ``w`` [H, K, N]; with ``gate`` (float32
    rows, column ``gate_col + h``) the head's output is multiplied by the sigmoid of its gate; ``gate_each``: every
    element has a gate of its own (column ``gate_col + h * N + n``)."""
    _cuda_contig(x, w, out)
    _f32(gate)
    T = x.shape[0]
    _need(x.shape == (T, H * K) and w.shape == (H, K, N) and out.shape == (T, H * N), "head_project: shapes")
    _need(gate is None or (gate.stride(-1) == 1 and gate.shape[0] == T and gate.shape[1] >= gate_col + (H * N if gate_each else H)),
          "head_project: gate rows")
    _check(lib().nv_head_project(_p(x), dt(x), _p(w), dt(w), _p(gate), (gate.stride(0) if gate is not None else 0), gate_col,
                                 _p(out), dt(out), T, H, K, N, (1 if gate_each else 0), _stream()), "head_project")


# ----------------------------------------------------------------------------- fast products
_num_sms = None


def head_gate(x, gate, gate_col: int, out, H: int, N: int, gate_each: bool = False) -> None:
    """``out[t, h, :] = x[t, h, :] * sigmoid(gate[t, gate_col + h])`` for float32 ``x`` [T, H * N] and float32 ``gate``
    rows; ``out`` in either dtype; ``gate_each``: element n of head h has the gate ``gate_col + h * N + n``."""
    _cuda_contig(x, out)
    _f32(x, gate)
    T = x.shape[0]
    _need(x.shape == (T, H * N) and out.shape == x.shape and gate.stride(-1) == 1 and gate.shape[0] == T
          and gate.shape[1] >= gate_col + (H * N if gate_each else H), "head_gate: shapes")
    _check(lib().nv_head_gate(_p(x), _p(gate), gate.stride(0), gate_col, _p(out), dt(out), T, H, N,
                              (1 if gate_each else 0), _stream()),
           "head_gate")


def stream_mix_norm(x, streams: int, *, branch=None, mix=None, carry=None, write=None, read=None, norm=None,
                    out=None, out32=None) -> None:
    """The copies of the residual stream ``x`` [T, streams * H] (float32, copy after copy inside a row), in one launch:

    1. with a pending sublayer output y (``branch`` [T, H] float32, or ``mix`` = (rows, index, weight, dense, None):
       ``y = dense + sum_r weight[:, r] * rows[index[:, r]]``) every copy d becomes
       ``sum_c carry[c, d] * x_c + write[d] * y`` (``carry`` [streams, streams] indexed [from, to], ``write``
       [streams]); with one copy and neither tensor ``x += y``;
    2. ``u = sum_d read[d] * x_d`` (``read`` None: the plain sum of the copies);
    3. ``norm`` = (alpha [1], gain [H], shift [H]), all float32: ``tanh(alpha * u) * gain + shift``; None: u itself;
    4. the result goes to ``out`` (float32 or bfloat16) and / or ``out32``; with neither, only step 1 is done."""
    _need(x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and x.dim() == 2 and x.shape[1] % streams == 0,
          "stream_mix_norm: the copies are float32 [T, streams * H]")
    T, H = x.shape[0], x.shape[1] // streams
    rows = index = weight = dense = None
    R = 0
    if mix is not None:
        _need(branch is None, "stream_mix_norm: one form of the pending output at a time")
        rows, index, weight, dense, gate = mix
        _need(gate is None, "stream_mix_norm: a gated dense term is not taken")
        R = index.shape[1]
        _need(R <= STREAM_MAX_MIX, f"stream_mix_norm: at most {STREAM_MAX_MIX} rows are mixed per token")
        _need(rows.dtype == torch.float32 and rows.shape[1] == H and rows.is_contiguous() and index.dtype == torch.int32
              and weight.dtype == torch.float32 and index.shape == (T, R) and weight.shape == (T, R)
              and index.is_contiguous() and weight.is_contiguous(), "stream_mix_norm: mix shapes")
    for t_ in (branch, dense, out32):
        _need(t_ is None or (t_.dtype == torch.float32 and t_.shape == (T, H) and t_.is_contiguous()),
              "stream_mix_norm: float32 [T, H] rows")
    _need(out is None or (out.shape == (T, H) and out.is_contiguous()), "stream_mix_norm: out is [T, H]")
    _need((carry is None) == (write is None), "stream_mix_norm: carry and write come together")
    if carry is not None:
        _need(carry.dtype == torch.float32 and carry.shape == (streams, streams) and carry.is_contiguous()
              and write.dtype == torch.float32 and write.numel() == streams, "stream_mix_norm: carry / write shapes")
    _need(read is None or (read.dtype == torch.float32 and read.numel() == streams), "stream_mix_norm: read shape")
    alpha = gain = shift = None
    if norm is not None:
        alpha, gain, shift = norm
        _f32(alpha, gain, shift)
        _need(alpha.numel() == 1 and gain.numel() == H and shift.numel() == H, "stream_mix_norm: norm shapes")
    if H % 4 == 0:
        for t_ in (x, branch, rows, dense, out, out32, gain, shift):
            _need(t_ is None or t_.data_ptr() % 16 == 0, "stream_mix_norm: rows must start on 16-byte boundaries")
    _check(lib().nv_stream_mix_norm(_p(x), T, streams, H, _p(branch), _p(rows), _p(index), _p(weight), R, _p(dense),
                                    _p(carry), _p(write), _p(read), (0 if norm is None else 1), _p(alpha), _p(gain),
                                    _p(shift), _p(out), (dt(out) if out is not None else 0), _p(out32), _stream()),
           "stream_mix_norm", nbytes=4.0 * T * H * (2 * streams + 2))


STREAM_MAX_STREAMS = 8
STREAM_MAX_MIX = 64


def scale_softcap(z, scale: float, cap: float) -> None:
    """``z = cap * tanh(scale * z / cap)`` in place (``cap`` <= 0: ``scale * z``); float32."""
    _need(z.dtype == torch.float32 and z.is_cuda and z.is_contiguous(), "scale_softcap: float32 values")
    _check(lib().nv_scale_softcap(_p(z), z.numel(), float(scale), float(cap), _stream()), "scale_softcap")


def num_sms() -> int:
    global _num_sms
    if _num_sms is None:
        _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _num_sms


def _tma_ok(t) -> bool:
    return (t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(st % 8 == 0 for st in t.stride()[:-1]))


def gemm_fast_usable(a, w, out, *, bias=None, a_rows=None, swiglu=False, grouped=False) -> bool:
    """Whether the tensor-core product takes these operands; the plain product takes all.

    Both operands bfloat16 with K a multiple of 8 (TMA moves 16-byte units), output float32 or
    bfloat16."""
    if not (_tma_ok(a) and _tma_ok(w) and w.is_contiguous()):
        return False
    if a.shape[-1] % 8 or out.dtype not in _DT or out.stride(-1) != 1:
        return False
    return True


SKINNY_MAX_ROWS = 32               # without SwiGLU; 8 with it
GROUPED_SPLIT_MAX_PAIRS = 16       # grouped products of at most this many (row, expert) pairs may split K


def skinny_usable(a, w, rows: int, swiglu: bool = False) -> bool:
    """Whether the weight-streaming product for a handful of rows (skinny_gemm.cu) takes these operands."""
    return (1 <= rows <= (8 if swiglu else SKINNY_MAX_ROWS) and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.stride(-1) == 1 and w.is_contiguous() and a.shape[-1] % 32 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(a, w, out, *, bias=None, swiglu=False, rows=None, err=None, act=None) -> None:
    """``out[:rows] = a[:rows] @ w.T (+ bias)`` for at most 32 rows (8 with ``swiglu``; default: all rows of ``a``),
    by streaming ``w`` once; ``swiglu`` as in ``gemm_plain``."""
    _cuda_contig(w, bias)
    K = a.shape[-1]
    rows_w = w.shape[0]
    N = rows_w // 2 if swiglu else rows_w
    R = a.shape[0] if rows is None else rows
    _need(skinny_usable(a, w, R, swiglu), "skinny product: operands or row count not supported")
    _need(w.dim() == 2 and w.shape[1] == K and out.shape[1] == N and out.stride(1) == 1 and out.shape[0] >= R,
          "skinny product: shapes")
    _need(bias is None or (not swiglu and bias.numel() == N), "skinny product: bias")
    _check(lib().nv_skinny_gemm(_p(a), a.stride(0), R, _p(w), N, K,
                                _p(bias), (dt(bias) if bias is not None else 0), _p(out), dt(out),
                                out.stride(0), _epilogue(swiglu, act), *_act_numbers(act), _stream()),
           f"skinny_gemm N={rows_w} K={K}", 0.0, float(w.element_size() * rows_w * K))


def grouped_token_tile(TK: int, E: int, swiglu: bool = False) -> int:
    """Token tile of the grouped tensor-core product for TK (row, expert) pairs over E experts: the most rows of
    one expert that a CTA takes at once.  The product's instruction is as wide as a tile's rows need (in steps
    of 16) and so are its token loads (in boxes of 64 rows), so a short last tile of an expert is cheap.  Tiles
    of 256 rows are accepted but lose (one accumulator set instead of two: 23.9 against 20.5 ms for a prompt of
    2,048 tokens).  ``swiglu`` lets the two products of an expert layer choose differently; they agree."""
    avg = (TK + E - 1) // E
    if avg <= 12:
        return 16
    if avg <= 24:
        return 32
    return 128 if avg >= 96 else 64


def permute_rows(src, rows, R=None):
    """bfloat16 rows of ``src`` gathered in the order of ``rows``."""
    R = rows.numel() if R is None else R
    dst = torch.empty((R, src.shape[1]), dtype=src.dtype, device=src.device)
    _check(lib().nv_permute_rows_bf16(_p(src), _p(rows), _p(dst), R, src.shape[1], _stream()),
           "permute_rows")
    return dst


def gemm_fast(a, w, out, *, bias=None, a_rows=None, swiglu=False, M=None, err=None, splits=None, act=None) -> None:
    """Tensor-core form of ``gemm_plain`` (dense)."""
    if a_rows is not None:
        a = permute_rows(a, a_rows, M)
    M = a.shape[0] if M is None else M
    K = a.shape[1]
    rows_w = w.shape[0]
    N = rows_w // 2 if swiglu else rows_w
    L = lib()
    n_tile = L.nv_tc_gemm_token_tile(M, (1 if swiglu else 0))
    if splits is None:
        splits = L.nv_tc_gemm_splits(M, N, K, n_tile, num_sms())
    scratch = None
    if splits > 1:
        scratch = torch.empty((splits, M, 2 * N if swiglu else N), dtype=torch.float32, device=a.device)
    _check(L.nv_tc_gemm(_p(a), a.stride(0), M, _p(w), rows_w, N, K,
                        _p(bias), (dt(bias) if bias is not None else 0), _p(out), dt(out),
                        out.stride(0), _epilogue(swiglu, act), n_tile, splits,
                        _p(scratch), _p(None), _p(None), _p(None), _p(None), 0, 0,
                        _p(err.t if err is not None else _global_err().t), _early(), 0, 0,
                        0, _p(None), 0, *_act_numbers(act), 0, 0, 0, _stream()), f"tc_gemm N={rows_w} K={K}", 2.0 * M * rows_w * K,
           w.element_size() * rows_w * K + a.element_size() * M * K + out.element_size() * M * N)


def gemm_fast_grouped(a, w, out, align, *, a_rows=None, swiglu=False, err=None, tiles=None, tiles_ready=False,
                      x_rows=None, max_ctas: int = 0, counter=None, act=None) -> None:
    """Tensor-core form of the grouped ``gemm_plain``; ``tiles`` (a TileList of ``align``) picks the token tile.

    ``x_rows`` = (sub, mod): a tile whose outputs are rows r.. takes rows ``(r - sub) % mod``.. of ``a`` (several
    experts that all take the same few rows, their outputs one segment after the other).

    ``max_ctas`` > 0 caps the grid, for a product that runs beside other kernels and must leave them room.
    ``counter`` (one int32 on the device, 0 between launches, used by one product at a time): the CTAs take their
    tiles from it instead of by position, so a CTA that starts late takes fewer.

    ``tiles_ready``: the tile lists were complete before the kernel that precedes this product on the stream
    started, so the product may start beside that kernel and fetch its first weights (it reads the lists at
    once).  With ``a_rows`` that holds by itself: the row copy comes between the routing and the product."""
    if a_rows is not None:
        a = permute_rows(a, a_rows, align.TK)
        tiles_ready = True
    K = a.shape[1]
    E, rows_w = w.shape[0], w.shape[1]
    N = rows_w // 2 if swiglu else rows_w
    tl = tiles if tiles is not None else align.primary
    _need(tl.tile_m in (16, 32, 64, 128, 256), "grouped product: token tile must be 16, 32, 64, 128 or 256")
    x_sub, x_mod = x_rows if x_rows is not None else (0, 0)
    _need(out.shape[0] >= align.TK and (x_mod or a.shape[0] <= align.TK), "grouped product: row counts")
    # One or two rows: the list has few tiles (an expert's matrix is a dozen tiles of 128 features), which would
    # leave most multiprocessors idle and each CTA with a long stream of its own; K is then split as in a small
    # dense product and a finishing kernel adds the parts.  (Measured per decode step: batch 1 492 -> 504 tokens/s;
    # with more rows the parts' traffic and the crowding of the other stream's product cost more than the split
    # gains: batch 4 1,464 -> 1,420, batch 64 6,219 -> 5,300.)
    splits, scratch = 1, None
    k_steps = (K + 63) // 64
    ctas = tl.max_tiles * ((N + 127) // 128)
    if counter is None and align.TK <= GROUPED_SPLIT_MAX_PAIRS and ctas < num_sms() and k_steps >= 8:
        splits = max(1, min(2 * num_sms() // ctas, k_steps // 4, 16))
        if splits > 1:
            scratch = torch.empty((splits, align.TK, 2 * N if swiglu else N), dtype=torch.float32, device=a.device)
    _check(lib().nv_tc_gemm(_p(a), a.stride(0), a.shape[0], _p(w), E * rows_w, N,
                            K, _p(None), 0, _p(out), dt(out), out.stride(0),
                            _epilogue(swiglu, act), tl.tile_m, splits, _p(scratch), _p(tl.tile_expert),
                            _p(tl.tile_row0), _p(tl.tile_rows), _p(tl.num_tiles), tl.max_tiles,
                            rows_w, _p(err.t if err is not None else _global_err().t),
                            (_early() if tiles_ready else 0), x_sub, x_mod, max_ctas,
                            _p(counter), align.TK, *_act_numbers(act), 0, 0, 0, _stream()),
           f"tc_gemm_grouped N={rows_w} K={K}")


class HeadTiles:
    """The fixed tile list of a product per head over ``T`` rows that hold their ``H`` heads side by side: one tile
    per (token tile, head), the heads of a token tile next to one another so that the CTAs that run together read
    the same rows."""

    def __init__(self, T: int, H: int, device, tile_m: int = 128):
        self.T, self.H, self.tile_m = T, H, tile_m
        heads, row0, rows = [], [], []
        for r in range(0, T, tile_m):
            for h in range(H):
                heads.append(h)
                row0.append(r)
                rows.append(min(tile_m, T - r))
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tiles = len(heads)
        self.tile_expert = torch.tensor(heads, **i32)
        self.tile_row0 = torch.tensor(row0, **i32)
        self.tile_rows = torch.tensor(rows, **i32)
        self.num_tiles = torch.tensor([len(heads)], **i32)


def gemm_fast_heads_usable(x, w, out, K: int) -> bool:
    return bool(_tma_ok(x) and _tma_ok(w) and w.is_contiguous() and K % 8 == 0 and out.dtype in _DT
                and out.stride(-1) == 1 and x.shape[0] > 0)


def gemm_fast_heads(x, w, out, tiles: HeadTiles, x_step: int, o_step: int, err=None) -> None:
    """``out[t, h * o_step + n] = sum_k x[t, h * x_step + k] * w[h, n, k]`` for k < K = ``w.shape[2]``: one product per
    head on the tensor cores in a single launch, over bfloat16 rows that hold their heads side by side (``x_step``
    columns apart; a head's K columns may be the first of its block).  ``w`` is [H, N, K]; ``tiles``: a ``HeadTiles``
    for these rows."""
    H, N, K = w.shape
    T = x.shape[0]
    _need(gemm_fast_heads_usable(x, w, out, K) and tiles.T == T and tiles.H == H, "per-head product: operands")
    _need(x_step % 8 == 0 and x.shape[1] >= (H - 1) * x_step + K and out.shape[0] >= T
          and out.shape[1] >= (H - 1) * o_step + N, "per-head product: shapes")
    _check(lib().nv_tc_gemm(_p(x), x.stride(0), T, _p(w), H * N, N, K, _p(None), 0, _p(out), dt(out), out.stride(0),
                            0, tiles.tile_m, 1, _p(None), _p(tiles.tile_expert), _p(tiles.tile_row0),
                            _p(tiles.tile_rows), _p(tiles.num_tiles), tiles.max_tiles, N,
                            _p(err.t if err is not None else _global_err().t), 0, 0, 0, 0, _p(None), T, 0.0, 0.0,
                            x_step, o_step, x.shape[1], _stream()),
           f"tc_gemm_heads N={N} K={K}", 2.0 * T * H * N * K)


_dependent_launch = 1


def set_dependent_launch(on: bool) -> None:
    """Whether a step's kernels are launched as programmatic dependents of one another (the default) or the
    ordinary way; for comparisons."""
    global _dependent_launch
    _dependent_launch = 1 if on else 0
    lib().nv_set_dependent_launch(_dependent_launch)


def _early() -> int:
    return _dependent_launch


_gerr = None


def _global_err() -> "ErrorFlag":
    global _gerr
    if _gerr is None:
        _gerr = ErrorFlag(torch.device("cuda", torch.cuda.current_device()))
    return _gerr
