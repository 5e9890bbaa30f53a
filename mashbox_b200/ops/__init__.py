"""Python faces of the hand-written CUDA kernels (mashbox_b200/csrc) and of the one library routine the engine uses.

Every function works on CUDA tensors, launches on torch's current stream and raises KernelError when the kernel
refuses the sizes.  There is no CPU or library fallback for a kernel: if the extension cannot be built or no GPU is
there, the call fails.  The only library call is the bf16 matrix product (cuBLAS through torch.mm), which stands where
the reference engine, too, hands its contractions to a library (src/mashbox/ops/dense16.py:73-75).
"""
import ctypes

import torch

from ..errors import KernelError
from .build import load_library

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

# bf16 products accumulate in float32 all the way: no reduced-precision reduction inside the library
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False

DEVICE_ERRORS = {1: "a token id outside the vocabulary", 2: "a position whose cache page the block table does not hold",
                 3: "a page id outside the cache pool", 4: "a bounded wait inside a kernel ran out"}


def _suffix(dtype):
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"no kernel for dtype {dtype}")


def _p(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    # the current stream's handle; torch.cuda.current_stream() costs several microseconds a call, a tenth of the host's
    # time in a step of two hundred launches, the raw accessor next to nothing
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("mashbox_b200 kernels run on CUDA tensors only; there is no CPU fallback")


COUNTERS = {"launches": 0}      # launches of this package's own kernels (a graph replay adds what it captured)


def _check(code, what):
    if code == 0:
        COUNTERS["launches"] += 1
        return
    if code == -2:
        raise KernelError(f"{what}: the kernel does not take these sizes")
    if code == -6:
        raise KernelError(f"{what}: the driver refused a tensor map")
    raise KernelError(f"{what}: CUDA error {code} at launch")


# Scratch that the faces below keep per device (partial sums, counters, reduction buffers) is made once and grows
# when a larger problem comes.  A captured graph holds the addresses it was captured with, so whoever replays graphs
# must capture again after a growth: scratch_generation() changes whenever any such buffer was replaced.
_scratch = {"generation": 0}


def scratch_generation():
    return _scratch["generation"]


# Programmatic dependent launch along the chain of kernels of a small step: a kernel of these libraries may start while
# the kernel before it in the stream still runs, sets itself up (the weight-streaming products send for their first
# weights), and waits for that kernel by itself before it touches anything a kernel writes.  One switch per library,
# set through set_pdl(); the engine's option "pdl" turns it on.
PDL = {"on": False}
_PDL_SETTERS = {"gemm_stream": "mb_gemm_stream_set_pdl", "elementwise": "mb_elementwise_set_pdl",
                "attention_tma": "mb_attn_tma_set_pdl"}
_pdl_applied = {}


def _apply_pdl(lib):
    name = _PDL_SETTERS.get(lib)
    if name is not None and _pdl_applied.get(lib) != PDL["on"]:
        f = getattr(load_library(lib), name, None)
        if f is not None:
            f.argtypes = [c_int]
            f(1 if PDL["on"] else 0)
        _pdl_applied[lib] = PDL["on"]


def set_pdl(on):
    PDL["on"] = bool(on)
    for lib in list(_pdl_applied):
        _apply_pdl(lib)


_fn_cache = {}


def _fn(lib, name, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        _pdl_applied.setdefault(lib, None)
        _apply_pdl(lib)
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


def new_error_word(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


_error_words = {}


def error_word(device):
    """The one error word per device that kernels without a caller-supplied word report to (the engine's step function
    uses it for all its kernels, so one read after a step sees every report)."""
    key = str(torch.device(device))
    if key not in _error_words:
        _error_words[key] = new_error_word(device)
    return _error_words[key]


def check_error_word(err):
    """Reads the device error word (a synchronisation) and raises if a kernel left a code there."""
    code = int(err.item())
    if code:
        err.zero_()
        raise KernelError("a kernel reported: " + DEVICE_ERRORS.get(code, f"code {code}"))


# ------------------------------------------------------------------------------------------------ elementwise
def embed(tokens, table, x, err):
    """x[n] = table[tokens[n]] into the float32 residual stream x (N, D)."""
    _cuda(tokens, table, x)
    N, D = x.shape
    f = _fn("elementwise", "mb_embed_" + _suffix(table.dtype),
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(tokens), _p(table), _p(x), N, D, table.shape[0], _p(err), _stream()), "embed")


def add_rmsnorm(x, delta, delta_bias, weight, eps, out, rows=None):
    """v = x (+ delta (+ delta_bias)); written back to x unless rows is given; out = v * rsqrt(mean(v^2)+eps) * weight.
    x (N, D) float32; delta (N, D) and out in the activation dtype; weight, delta_bias float32; rows int32 indexes."""
    _cuda(x, delta, weight, out, rows)
    D = x.shape[1]
    n_out = out.shape[0]
    f = _fn("elementwise", "mb_add_rmsnorm_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(delta_bias), _p(rows), _p(weight), float(eps), _p(out), n_out, D, _stream()),
           "add_rmsnorm")


def rope_kv_write(qkv, bias, positions, tok_seq, table, kpool, vpool, freqs, H, KV, HD, RD, pairing, page, num_pages,
                  err):
    """qkv (N, (H + 2 KV) HD): adds bias, rotates q in place, writes rotated k and v to their pages (kpool/vpool None:
    q only).  freqs (RD/2,) float32 angle per position step, None = no rotation; pairing 0 adjacent, 1 halves."""
    _cuda(qkv, positions, tok_seq, table, kpool, vpool, freqs)
    N = qkv.shape[0]
    f = _fn("elementwise", "mb_rope_kv_write_" + _suffix(qkv.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 8
            + [c_void_p, c_void_p])
    _check(f(_p(qkv), _p(bias), _p(positions), _p(tok_seq), _p(table), table.shape[1], _p(kpool), _p(vpool), _p(freqs),
             N, H, KV, HD, RD, pairing, page, num_pages, _p(err), _stream()), "rope_kv_write")


def patch_tokens(dst, src, pairs, n):
    """dst[pairs[2i]] = src[pairs[2i+1]] for i < n (int32 tensors on the device)"""
    _cuda(dst, src, pairs)
    f = _fn("elementwise", "mb_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(dst), _p(src), _p(pairs), int(n), _stream()), "patch_tokens")


def swiglu(gu, out):
    """gu (N, 2F) = [gate | up] -> out (N, F) = silu(gate) * up"""
    _cuda(gu, out)
    N, F = out.shape
    f = _fn("elementwise", "mb_swiglu_" + _suffix(out.dtype), [c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(gu), _p(out), N, F, _stream()), "swiglu")


# ------------------------------------------------------------------------------------------------ contractions
def linear(a, w, out=None, out_dtype=None):
    """a (N, K) @ w (M, K)^T -> (N, M).  float32: the package's own fixed-order FFMA kernel (no TF32, no tensor
    cores).  bfloat16: cuBLAS with float accumulation; out_dtype float32 keeps the accumulator's precision."""
    _cuda(a, w)
    N, K = a.shape
    M = w.shape[0]
    if a.dtype == torch.float32:
        if out is None:
            out = torch.empty((N, M), dtype=torch.float32, device=a.device)
        f = _fn("gemm_f32", "mb_gemm_f32", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(f(_p(a), _p(w), _p(out), N, M, K, _stream()), "gemm_f32")
        return out
    if tc5_supports(N, M, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want in (torch.bfloat16, torch.float32):
            return linear_tc5(a, w, out, "plain" if want == torch.bfloat16 else "float")
    if gemv_supports(N, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want == torch.bfloat16:      # the output head stays with the library
            return linear_gemv(a, w, out, "plain")
    if stream_supports(N, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16 and M % 8 == 0:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want in (torch.bfloat16, torch.float32):
            return linear_stream(a, w, out, "plain" if want == torch.bfloat16 else "float")
    if out_dtype is not None and out_dtype != a.dtype:
        r = torch.mm(a, w.t(), out_dtype=out_dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is not None:
        return torch.mm(a, w.t(), out=out)
    return torch.mm(a, w.t())


# The package's own tcgen05 product for prompt portions (128 tokens or more).  "swiglu": the fused gate/up product
# (measured 317 us against 310 + 33 us for the library product and the separate gate kernel at 2,048 tokens of the
# Llama-3.1-8B shape); "plain": every product (87 to 97 % of the library's speed, so off by default).
TC5 = {"swiglu": True, "plain": False}


def tc5_supports(N, M, K, mode="plain"):
    return TC5["swiglu" if mode == "swiglu" else "plain"] and N >= 128 and K >= 8 and K % 8 == 0 and M % 8 == 0


def linear_tc5(a, w, out, mode="plain"):
    """a (N, K) bf16, w (M, K) bf16 (mode "swiglu": (2M, K) = [gate rows | up rows]) -> out (N, M): bf16 for "plain" and
    "swiglu" (silu(gate) * up), float32 for "float".  TMA + tcgen05.mma with the accumulator in tensor memory."""
    _cuda(a, w, out)
    N, K = a.shape
    name = {"plain": "mb_gemm_tc5_bf16", "swiglu": "mb_gemm_tc5_swiglu_bf16", "float": "mb_gemm_tc5_f32out"}[mode]
    f = _fn("gemm_tc5", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(a), _p(w), _p(out), N, out.shape[1], K, _p(error_word(a.device)), _stream()), "gemm_tc5")
    return out


# Matrix-vector products (one warp per two rows of W, or a block per two long rows; no tensor core): the kernels take up
# to 4 tokens, the engine uses them where they beat the library, which is at ONE token.  Measured inside captured
# graphs on the Llama-3.1-8B shapes at one token, own / library: output product 10.8 / 13.0 us, QKV 12.2 / 11.7, down
# 21.2 / 24.9, fused gate/up + SwiGLU 39.0 / 39.2 + 2.3; at two tokens the arithmetic (bf16 to float conversions on
# the FMA pipe) already costs more than the stream.  GEMV[mode] = the most tokens the engine gives the kernel (0: never);
# "fused": the forms that normalise the residual stream themselves or add their product into it (see small_fused_supports).
# A limit of -1 leaves the choice to the width of the product's input (GEMV_AUTO: the matrix-vector kernels up to that
# many tokens below that width, else the weight-streaming products).  One request, 128 new tokens after 32 of prompt,
# through Engine.admit/step (python bench.py --workload 1b-single and the like), matrix-vector / streaming: Llama-3.2-1B
# shape (width 2,048) 1,378 / 987 tokens/s, Llama-3.2-3B shape (3,072) 605 / 498, Falcon3-1B shape (2,048) 1,047 / 765,
# Llama-3.1-8B shape (4,096) 328 / 315 (the same at 8,192 tokens of context: 3.35 ms a step either way): the advantage
# shrinks with the width (+40 %, +21 %, +4 %), so the line for one token is drawn between 4,096 and 5,120.  At two
# tokens (2,048 of context) the 1B shape takes 0.88 / 0.91 ms a step, the 3B shape 1.98 / 1.88, the 8B shape 3.84 /
# 3.55; at three they are level, at four the streaming products win everywhere.
GEMV = {"swiglu": 1, "plain": 1, "fused": 1}
GEMV_AUTO = ((2560, 2), (4608, 1))            # (narrower than, tokens), the first line that applies


def _gemv_limit(mode, K):
    v = GEMV[mode]
    if v >= 0:
        return v
    if not PDL["on"]:
        return 1
    for width, tokens in GEMV_AUTO:
        if K < width:
            return tokens
    return 0


def gemv_supports(N, K, mode="plain"):
    return 1 <= N <= min(4, _gemv_limit("swiglu" if mode == "swiglu" else "plain", K)) and K >= 8 and K % 8 == 0


def linear_gemv_normed(x, norm_w, eps, w, out, mode="plain"):
    """x (N <= 4, K) float32 residual stream, norm_w (K) float32 -> out (N, M) bf16 = rmsnorm(x) W^T ("swiglu": W is
    (2M, K) and out = silu(gate) * up), the normalised row rounded to bf16 as the norm kernel would store it."""
    _cuda(x, norm_w, w, out)
    N, K = x.shape
    name = {"plain": "mb_gemv_normed_bf16", "swiglu": "mb_gemv_normed_swiglu_bf16"}[mode]
    f = _fn("gemv", name, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(norm_w), float(eps), _p(w), _p(out), N, out.shape[1], K, _stream()), "gemv_normed")
    return out


def linear_gemv_normed_qkv(x, norm_w, eps, w, out, bias, positions, tok_seq, table, kpool, vpool, freqs, H, KV, HD, RD,
                           pairing, page, num_pages, err):
    """x (N <= 4, K) float32 residual stream -> the fused q/k/v product of rmsnorm(x) with the rotate-and-store step in
    its epilogue: out (N, (H + 2 KV) HD) bf16 receives the rotated q heads, the rotated k and the v heads go into the
    pages of the tokens' positions (kpool None: dropped), as rope_kv_write would leave them."""
    _cuda(x, norm_w, w, out, bias, positions, tok_seq, table, kpool, vpool, freqs)
    N, K = x.shape
    f = _fn("gemv", "mb_gemv_normed_qkv_bf16",
            [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_void_p])
    _check(f(_p(x), _p(norm_w), float(eps), _p(w), _p(out), N, out.shape[1], K, _p(bias), _p(positions), _p(tok_seq),
             _p(table), table.shape[1], _p(kpool), _p(vpool), _p(freqs), H, KV, HD, RD, pairing, page, num_pages,
             _p(err), _stream()), "gemv_normed_qkv")
    return out


def linear_gemv_residual(a, w, x, bias=None):
    """x (N <= 4, M) float32 += a (N, K) bf16 @ w (M, K)^T (+ bias (M) float32), in place"""
    _cuda(a, w, x, bias)
    N, K = a.shape
    f = _fn("gemv", "mb_gemv_residual", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(a), _p(w), _p(x), _p(bias), N, x.shape[1], K, _stream()), "gemv_residual")
    return x


def linear_gemv(a, w, out, mode="plain"):
    """a (N <= 4, K) bf16, w (M, K) bf16 ("swiglu": (2M, K)) -> out (N, M): bf16, or float32 for mode "float"."""
    _cuda(a, w, out)
    N, K = a.shape
    name = {"plain": "mb_gemv_bf16", "swiglu": "mb_gemv_swiglu_bf16", "float": "mb_gemv_f32out"}[mode]
    f = _fn("gemv", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(a), _p(w), _p(out), N, out.shape[1], K, _stream()), "gemv")
    return out


# The weight-streaming products for steps of 2 to 16 tokens (gemm_stream.cu): W is cut into row tiles low enough that
# most SMs get one (no tile shared for the layer's own matrices), streamed by TMA, mma.sync on the tiles.  The product
# that ends a sublayer adds into the residual stream and leaves what the norm after it needs (sums of squares, rows
# times the norm's weight); the product after that norm runs on those rows and scales its sums by 1 / rms; gate/up has
# SwiGLU in its epilogue.  A layer is then six kernels instead of ten.  Measured inside captured graphs on the
# Llama-3.1-8B shapes at 8 tokens, own / library, us: output product with the residual add 11.4 / 12.0 (+ the add in the
# norm kernel), q/k/v of the normalised stream 12.0 / 11.9 + norm 3.8, gate/up with SwiGLU 40.6 / 40.2 + norm 3.8 + gate
# 2.3, down with the residual add 26.5 / 23.3; the whole decode step at batch 8 (the output head too): 1,720 tokens/s
# against 1,608 with the library's products.  STREAM["tokens"]: the most tokens the engine gives them (0: never).
STREAM = {"tokens": 16}


def configure(options):
    """Engine options that choose between this package's kernels, applied process-wide (the kernels' faces are module
    functions).  pdl (default on): programmatic dependent launch along the chain of kernels of a small step; with it
    the weight-streaming products take steps of one token too when the model is wide enough (GEMV_AUTO)
    (narrower models stay with the matrix-vector kernels, which are launched plainly: launched that way themselves
    they lost 0.7 ms a step on the 8B shape).
    gemv_tokens / stream_tokens: the most tokens of a step the matrix-vector / weight-streaming products take (0: never;
    gemv_tokens unset: by the width)."""
    pdl = bool(options.get("pdl", True))
    set_pdl(pdl)
    for k in GEMV:
        GEMV[k] = int(options["gemv_tokens"]) if "gemv_tokens" in options else (-1 if pdl else 1)
    STREAM["tokens"] = int(options.get("stream_tokens", 16))


_stream_scratch = {}


def stream_supports(N, K):
    return 1 <= N <= min(16, STREAM["tokens"]) and K >= 8 and K % 8 == 0


def _stream_buffers(device, M):
    """(workspace, counters) of the streaming products on this device: the partial sums of row tiles that blocks
    share, and a counter per row tile, zero between launches"""
    lib = load_library("gemm_stream")
    lib.mb_gemm_stream_workspace.restype = ctypes.c_longlong
    key = str(device)
    sc = _stream_scratch.get(key)
    tiles = (M + 31) // 32
    if sc is None or sc[1].numel() < tiles:
        sc = (torch.empty(lib.mb_gemm_stream_workspace(), dtype=torch.float32, device=device),
              torch.zeros(max(tiles, 8192), dtype=torch.int32, device=device))
        _stream_scratch[key] = sc
        _scratch["generation"] += 1
    return sc


def linear_stream(a, w, out, mode="plain", sums=None, eps=0.0):
    """a (N <= 16, K) bf16, w (M, K) bf16 ("swiglu": (2M, K)) -> out (N, M): bf16, or float32 for mode "float".
    sums (ceil(K / 32), 16) float32, if given: a holds rows of a residual stream times a norm's weight and sums the sums
    of squares of those rows by 32 columns, as linear_stream_residual leaves them; out is then the product of
    rmsnorm(x; weight, eps): 1 / rms scales the float sums of the product."""
    _cuda(a, w, out, sums)
    N, K = a.shape
    M = out.shape[1]
    ws, cnt = _stream_buffers(a.device, M)
    f = _fn("gemm_stream", "mb_gemm_stream", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(a), _p(sums), float(eps), _p(w), _p(out), N, M, K, {"plain": 0, "swiglu": 1, "float": 2}[mode], _p(ws),
             _p(cnt), _p(error_word(a.device)), _stream()), "gemm_stream")
    return out


def linear_stream_residual(a, w, x, bias=None, sums=None, next_w=None, scaled=None):
    """x (N <= 16, M) float32 += a (N, K) bf16 @ w (M, K)^T (+ bias (M) float32), in place.  What the norm that reads x
    next needs, on request: sums (ceil(M / 32), 16) float32 receives the sums of squares of the new rows by 32 columns,
    scaled (N, M) bf16 the new rows times that norm's weight next_w (M) float32."""
    _cuda(a, w, x, bias, sums, next_w, scaled)
    N, K = a.shape
    M = x.shape[1]
    ws, cnt = _stream_buffers(a.device, M)
    f = _fn("gemm_stream", "mb_gemm_stream_residual", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(a), _p(w), _p(x), _p(bias), N, M, K, _p(sums), _p(next_w), _p(scaled), _p(ws), _p(cnt),
             _p(error_word(a.device)), _stream()), "gemm_stream_residual")
    return x


# ---- what the parts call at few tokens: the matrix-vector kernels where they are enabled, else the streaming products.
# "held" is what the product that last added into the residual stream left for the norm after it (sums of squares by 32
# columns, rows times the norm's weight in bf16): the streaming products need it, the matrix-vector kernels read x.
def _use_gemv_fused(N, K):
    return 1 <= N <= min(4, _gemv_limit("fused", K)) and K % 8 == 0 and 8 <= K < 8192 and N * K * 2 <= 48 * 1024


def small_fused_supports(N, K, dtype):
    """True when a step of N tokens of width K can run its layers on the folded kernels: the product that follows a
    norm is the product of the normalised stream without a norm kernel (linear_small_normed), the product that ends a
    sublayer adds into the stream (linear_small_residual)."""
    return dtype == torch.bfloat16 and (_use_gemv_fused(N, K) or stream_supports(N, K))


def small_normed_needs_held(N, K):
    return not _use_gemv_fused(N, K)


def small_qkv_supports(N, K):
    """True when linear_small_normed_qkv takes this step (else: linear_small_normed, then rope_kv_write)"""
    return _use_gemv_fused(N, K)


def linear_small_normed(x, norm_w, eps, w, out, mode="plain", held=None):
    if _use_gemv_fused(*x.shape):
        return linear_gemv_normed(x, norm_w, eps, w, out, mode)
    sums, scaled = held
    return linear_stream(scaled, w, out, mode, sums, eps)


def linear_small_normed_qkv(x, norm_w, eps, w, out, *args):
    return linear_gemv_normed_qkv(x, norm_w, eps, w, out, *args)


def linear_small_residual(a, w, x, bias=None, sums=None, next_w=None, scaled=None):
    """-> True when sums and scaled were filled (see linear_stream_residual)"""
    if _use_gemv_fused(a.shape[0], x.shape[1]) and a.shape[1] % 8 == 0:
        linear_gemv_residual(a, w, x, bias)
        return False
    linear_stream_residual(a, w, x, bias, sums, next_w, scaled)
    return sums is not None and scaled is not None


def fused_swiglu_supports(N, F, K):
    return gemv_supports(N, K, "swiglu") or stream_supports(N, K) or tc5_supports(N, F, K, "swiglu")


def linear_swiglu(a, wgu, out):
    """a (N, K) bf16, wgu (2F, K) = [gate rows | up rows] -> out (N, F) = silu(a Wg^T) * (a Wu^T), one kernel: the
    tcgen05 product for prompt portions, the matrix-vector or the weight-streaming kernel for decode batches (where enabled).
    Only for shapes fused_swiglu_supports() takes."""
    _cuda(a, wgu, out)
    N, K = a.shape
    if tc5_supports(N, out.shape[1], K, "swiglu"):
        return linear_tc5(a, wgu, out, "swiglu")
    if gemv_supports(N, K, "swiglu"):
        return linear_gemv(a, wgu, out, "swiglu")
    if stream_supports(N, K):
        return linear_stream(a, wgu, out, "swiglu")
    raise KernelError("linear_swiglu: no fused kernel takes these sizes")


# ------------------------------------------------------------------------------------------------ attention
def attention_simple(q, q_stride, out, positions, tok_seq, table, kpool, vpool, H, KV, HD, page, num_pages, window,
                     scale, err):
    _cuda(q, out, positions, tok_seq, table, kpool, vpool)
    N = out.shape[0]
    f = _fn("attention_simple", "mb_attn_simple_" + _suffix(out.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7
            + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(positions), _p(tok_seq), _p(table), table.shape[1], _p(kpool), _p(vpool), N,
             H, KV, HD, page, num_pages, window or 0, float(scale), _p(err), _stream()), "attention_simple")


def attention_mma_supports(HD):
    """head sizes in steps of 16 up to 256 (16, 32, 64, 128 in one library, the others in a second one)"""
    return 16 <= HD <= 256 and HD % 16 == 0


def _mma_library(HD):
    return "attention_mma" if HD in (16, 32, 64, 128) else "attention_mma_wide"


def attention_mma(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                  table,
                  part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale, err):
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, part_base, table, part_o, part_ml)
    f = _fn(_mma_library(HD), "mb_attn_mma_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, 1 if decode else 0, _p(q_start),
             _p(q_len), _p(pos0), _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml), max_splits, H, KV,
             HD, page, num_pages, window or 0, float(scale), _p(err), _stream()), "attention_mma")


def attention_tma_supports(HD, page):
    return HD in (64, 128) and page in (8, 16, 32, 64)


_merge_counters = {}
MERGE_COUNTERS = 1 << 16


def attention_tma_merges(n_items, KV):
    """True when attention_tma can merge the splits of its items itself (it has a counter for every group)"""
    return n_items * KV <= MERGE_COUNTERS


def attention_tma_folds_rotation(G):
    """True when attention_tma can take the rotate-and-store step of a step of one-token sequences in (rope=...)"""
    return 1 <= G <= 16


_max_cluster = {}


def attention_tma_max_cluster(HD):
    """the most splits of a sequence whose blocks attention_tma can launch as one thread-block cluster (1: none)"""
    if HD not in _max_cluster:
        lib = load_library("attention_tma")
        lib.mb_attn_tma_max_cluster.argtypes = [c_int, c_int]
        lib.mb_attn_tma_max_cluster.restype = c_int
        _max_cluster[HD] = max(1, min(lib.mb_attn_tma_max_cluster(HD, 0), lib.mb_attn_tma_max_cluster(HD, 1)))
    return _max_cluster[HD]


_active_clusters = {}


def attention_tma_active_clusters(HD, cluster):
    """how many clusters of `cluster` blocks of attention_tma's decode form the device holds at the same time"""
    if (HD, cluster) not in _active_clusters:
        lib = load_library("attention_tma")
        lib.mb_attn_tma_active_clusters.argtypes = [c_int, c_int, c_int]
        lib.mb_attn_tma_active_clusters.restype = c_int
        _active_clusters[HD, cluster] = min(lib.mb_attn_tma_active_clusters(HD, r, cluster) for r in (0, 1))
    return _active_clusters[HD, cluster]


def attention_tma(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                  table, part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale, err, merge=False,
                  rope=None, cluster=0):
    """The same contract as attention_mma, with K/V tiles loaded by TMA (head sizes 64 and 128, pages of 8 to 64).
    merge: the last block of every split group merges the group's partial results and writes `out`, so no
    attention_merge is needed afterwards (only when attention_tma_merges(n_items, KV)).
    cluster = n > 1 (decode form): every sequence of the launch is cut into n splits and the blocks of a sequence and kv
    head are launched as one thread-block cluster whose results meet in shared memory (no partial buffers, no merge);
    n at most attention_tma_max_cluster(HD).
    rope = (bias or None, freqs or None, RD, pairing): the step's sequences bring ONE token each and q is the whole
    (N, (H + 2 KV) HD) output of the q/k/v product; the kernel does what rope_kv_write would have done before it (bias,
    rotation of q and k, k and v into the token's page) -- the same bits, one launch fewer.  q itself is not changed."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, part_base, table, part_o, part_ml)
    if cluster and cluster > 1:
        if not decode:
            raise KernelError("attention_tma: clusters are for the decode form")
        bias, freqs, RD, pairing = rope if rope is not None else (None, None, 0, 0)
        _cuda(bias, freqs)
        f = _fn("attention_tma", "mb_attn_tma_cluster_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_int] + [c_int] * 7 + [c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
                 _p(seq_row), _p(table), table.shape[1], int(cluster), H, KV, HD, page, num_pages, window or 0,
                 float(scale), _p(err), 1 if rope is not None else 0, _p(bias), _p(freqs), int(RD), int(pairing), _stream())
        if code == -6:
            raise KernelError("attention_tma: the driver refused the tensor map of the cache pool")
        _check(code, "attention_tma")
        return
    counters = None
    if merge:
        if not attention_tma_merges(n_items, KV):
            raise KernelError("attention_tma: more split groups than merge counters")
        key = str(q.device)
        if key not in _merge_counters:
            _merge_counters[key] = torch.zeros(MERGE_COUNTERS, dtype=torch.int32, device=q.device)
            _scratch["generation"] += 1
        counters = _merge_counters[key]
    if rope is not None:
        if not decode:
            raise KernelError("attention_tma: the rotation is folded into the decode form only")
        bias, freqs, RD, pairing = rope
        _cuda(bias, freqs)
        f = _fn("attention_tma", "mb_attn_tma_rope_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p, c_void_p,
                                                                                c_void_p, c_int, c_int, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
                 _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml), max_splits, H, KV, HD,
                 page, num_pages, window or 0, float(scale), _p(counters), _p(err), _p(bias), _p(freqs), int(RD),
                 int(pairing), _stream())
    else:
        f = _fn("attention_tma", "mb_attn_tma_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, 1 if decode else 0, _p(q_start),
                 _p(q_len), _p(pos0), _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml),
                 max_splits, H, KV, HD, page, num_pages, window or 0, float(scale), _p(counters), _p(err), _stream())
    if code == -6:
        raise KernelError("attention_tma: the driver refused the tensor map of the cache pool")
    _check(code, "attention_tma")


def attention_tc5_supports(HD, page):
    return HD in (64, 128) and page in (8, 16, 32, 64, 128)


def attention_tc5_rows():
    """packed query rows of one work item of the tcgen05 attention kernel"""
    lib = load_library("attention_tc5")
    lib.mb_attn_tc5_rows.restype = c_int
    return lib.mb_attn_tc5_rows()


def attention_tc5(q, q_stride, out, kpool, vpool, items, n_items, q_start, q_len, pos0, seq_row, table, H, KV, HD, page,
                  num_pages, window, scale, err):
    """Prompt-form attention on tcgen05: items are (sequence, tile of attention_tc5_rows() packed rows, 0, 1); head
    sizes 64 and 128."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, seq_row, table)
    f = _fn("attention_tc5", "mb_attn_tc5_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int] + [c_int] * 6 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
             _p(seq_row), _p(table), table.shape[1], H, KV, HD, page, num_pages, window or 0, float(scale),
             _p(err), _stream()), "attention_tc5")


def attention_merge(part_o, part_ml, part_tok, n_part, out, H, HD, max_splits):
    _cuda(part_o, part_ml, part_tok, out)
    f = _fn("attention_mma", "mb_attn_merge_bf16",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(part_o), _p(part_ml), _p(part_tok), n_part, _p(out), H, HD, max_splits, _stream()), "attention_merge")


# ------------------------------------------------------------------------------------------------ sampling
def sample_params_size():
    lib = load_library("sampling")
    lib.mb_sample_params_size.restype = c_int
    return lib.mb_sample_params_size()


_sample_scratch = {}


def sample(logits, work, params, cnt, seen, n_rows, out, any_cut=True, keep_work=True):
    """logits (R, V) float32; work (n_rows, V) float32 scratch; params: uint8 tensor of n_rows packed RowParams;
    cnt (slots, V) int32 / seen (slots, V) uint8 penalty state or None; out (n_rows,) int32.  any_cut: False when no
    row has a top_k, top_p or min_p (the kernel that finds the cuts is skipped).  keep_work: leave the processed
    logits after the cuts (cut values -inf) in `work`, which costs a write of every row."""
    _cuda(logits, work, params, cnt, seen, out)
    key = str(logits.device)
    sc = _sample_scratch.get(key)
    if sc is None or sc[0].shape[0] < n_rows * 32:
        cap = max(n_rows, 64)
        sc = (torch.empty(cap * 32, dtype=torch.float32, device=logits.device),
              torch.empty(cap * 32, dtype=torch.int32, device=logits.device),
              torch.empty(cap * 2, dtype=torch.int32, device=logits.device))
        _sample_scratch[key] = sc
        _scratch["generation"] += 1
    f = _fn("sampling", "mb_sample_fast", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), _p(work), _p(params), _p(cnt), _p(seen), n_rows, logits.shape[1], _p(sc[2]), _p(sc[0]), _p(sc[1]),
             _p(work) if keep_work else None, 1 if any_cut else 0, _p(out), _stream()), "sample")


def sample_one_kernel(logits, work, params, cnt, seen, n_rows, out):
    """The same sampler as one kernel with a block per row that bisects the whole row (a millisecond for a batch at a
    vocabulary of 128k): what the entry point without allocations runs, kept callable for comparison."""
    _cuda(logits, work, params, cnt, seen, out)
    f = _fn("sampling", "mb_sample", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), _p(work), _p(params), _p(cnt), _p(seen), n_rows, logits.shape[1], _p(out), _stream()), "sample")


_argmax_scratch = {}


def argmax(logits, out):
    """out[r] = the lowest index of the maximum of row r"""
    _cuda(logits, out)
    n = logits.shape[0]
    key = str(logits.device)
    sc = _argmax_scratch.get(key)
    if sc is None or sc[0].shape[0] < n * 32:
        sc = (torch.empty(max(n, 64) * 32, dtype=torch.float32, device=logits.device),
              torch.empty(max(n, 64) * 32, dtype=torch.int32, device=logits.device))
        _argmax_scratch[key] = sc
        _scratch["generation"] += 1
    f = _fn("sampling", "mb_argmax", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), n, logits.shape[1], _p(sc[0]), _p(sc[1]), _p(out), _stream()), "argmax")


def penalty_fill(cnt_row, seen_row, tokens, n_prompt, n_total, V):
    _cuda(cnt_row, seen_row, tokens)
    f = _fn("sampling", "mb_penalty_fill", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(cnt_row), _p(seen_row), _p(tokens), n_prompt, n_total, V, _stream()), "penalty_fill")


# ------------------------------------------------------------------------------------------------ tracing
def logit_trace(logits, out):
    """logits (R, V) float32 contiguous -> out (R, 2) int32: per row the order-independent hash
    sum(bits(lg[v]) * (2 v + 1)) mod 2^32 and the bits of the float32 gap between the two largest logits
    (src/mashbox/runtime/engine.py:80-89)."""
    _cuda(logits, out)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("logit_trace: float32 contiguous logits only")
    f = _fn("trace", "mb_logit_trace", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), logits.shape[0], logits.shape[1], _p(out), _stream()), "logit_trace")


def read_logit_trace(pairs):
    """int32 (R, 2) as logit_trace writes it (any device or a numpy array) -> [(hash, gap)] with hash in 0..2^32-1"""
    import numpy as np
    a = np.ascontiguousarray(pairs.cpu().numpy() if hasattr(pairs, "cpu") else pairs, dtype=np.int32).reshape(-1, 2)
    return [(int(h), float(g)) for h, g in zip(a[:, 0].view(np.uint32), a[:, 1].copy().view(np.float32))]
