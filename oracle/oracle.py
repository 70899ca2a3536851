"""ctypes/numpy front of the CPU oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the
library never does.  bf16 tensors are numpy uint16 arrays of bit patterns.  PARITY UNPINNED: the
reference ships no golden vectors for this path (see the header of oracle.c).
"""
import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _cpu_tag():
    """Digest of this host's CPU feature flags: the library is built -march=native, so a build made
    on another kind of CPU must not be loaded here."""
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


TAG = _cpu_tag()
LIB = os.path.join(HERE, f"liboracle_{TAG}.so")

UNARY = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "relu": 4, "sigmoid": 5, "exp": 6}
PAIR = {"none": 0, "swiglu": 1, "geglu": 2, "rope": 3, "swap": 4}

_lib = None


def build(force=False):
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, f"TAG={TAG}", "-B" if force else "-s"],
                              stdout=subprocess.DEVNULL)
    return LIB


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.xo_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().xo_num_threads()


def set_num_threads(n):
    """OpenMP threads the oracle's loops use from now on (launchers such as torch.distributed.run
    export OMP_NUM_THREADS=1, which would otherwise stick)."""
    lib().xo_set_num_threads(int(n))


def f32_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().xo_f32_to_bf16(_p(x), _p(out), C.c_int64(x.size))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().xo_bf16_to_f32(_p(x), _p(out), C.c_int64(x.size))
    return out


def gemm_bf16(A, B):
    """A [M,K], B [K,N] uint16 bf16 bits -> float32 [M,N], fp32 accumulation."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    Cm = np.empty((M, N), dtype=np.float32)
    lib().xo_gemm_bf16_f32(_p(A), _p(B), _p(Cm), M, N, K)
    return Cm


def gemm_s8(A, B):
    """A [M,K], B [K,N] int8 -> exact int32 [M,N]."""
    A = np.ascontiguousarray(A, dtype=np.int8)
    B = np.ascontiguousarray(B, dtype=np.int8)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    Cm = np.empty((M, N), dtype=np.int32)
    lib().xo_gemm_s8_s32(_p(A), _p(B), _p(Cm), M, N, K)
    return Cm


def epilogue(acc, *, residual=None, row=None, col=None, bias=None, unary="none", pair="none",
             cos_sin=None, cos_sin_period=0, compact=False, want_aux=False, want_f32=False):
    """Runs the flat epilogue program on an accumulator [M,N] (float32 or int32).

    Returns bf16 bits [M,N] (or [M,N/2] when compact); with want_aux also the bf16 aux store;
    with want_f32 also the unrounded fp32 result."""
    if acc.dtype == np.int32:
        a = np.empty(acc.shape, dtype=np.float32)
        lib().xo_s32_to_f32(_p(np.ascontiguousarray(acc)), _p(a), C.c_int64(acc.size))
        acc = a
    acc = np.ascontiguousarray(acc, dtype=np.float32)
    M, N = acc.shape
    n_out = N // 2 if compact else N
    out = np.empty((M, n_out), dtype=np.uint16)
    outf = np.empty((M, n_out), dtype=np.float32) if want_f32 else None
    aux = np.empty((M, N), dtype=np.uint16) if want_aux else None
    f = lambda v: None if v is None else np.ascontiguousarray(v, dtype=np.float32)
    residual = None if residual is None else np.ascontiguousarray(residual, dtype=np.uint16)
    row, col, bias, cos_sin = f(row), f(col), f(bias), f(cos_sin)
    cs_ld = 0 if cos_sin is None else cos_sin.shape[1]
    lib().xo_epilogue(_p(acc), M, N, _p(residual), C.c_int64(N), _p(aux), C.c_int64(N), _p(row),
                      _p(col), _p(bias), UNARY[unary], PAIR[pair], _p(cos_sin), C.c_int64(cs_ld),
                      int(cos_sin_period), int(bool(compact)), _p(out), C.c_int64(n_out), _p(outf))
    res = [out]
    if want_aux:
        res.append(aux)
    if want_f32:
        res.append(outf)
    return res[0] if len(res) == 1 else tuple(res)


def preset_k1(acc, scale):
    M, N = acc.shape
    out = np.empty((M, N), np.uint16)
    lib().xo_preset_k1(_p(np.ascontiguousarray(acc, np.float32)), _p(np.ascontiguousarray(scale, np.float32)), M, N, _p(out))
    return out


def preset_k2(acc, scale, geglu=False):
    M, N = acc.shape
    out = np.empty((M, N), np.uint16)
    lib().xo_preset_k2(_p(np.ascontiguousarray(acc, np.float32)), _p(np.ascontiguousarray(scale, np.float32)), M, N, int(geglu), _p(out))
    return out


def preset_k4(acc, scale, cos_sin):
    M, N = acc.shape
    out = np.empty((M, N), np.uint16)
    s = None if scale is None else np.ascontiguousarray(scale, np.float32)
    lib().xo_preset_k4(_p(np.ascontiguousarray(acc, np.float32)), _p(s), _p(np.ascontiguousarray(cos_sin, np.float32)), M, N, _p(out))
    return out


def preset_k0a(acc, residual, gamma):
    M, N = acc.shape
    out = np.empty((M, N), np.uint16)
    lib().xo_preset_k0a(_p(np.ascontiguousarray(acc, np.float32)), _p(np.ascontiguousarray(residual, np.uint16)),
                        _p(np.ascontiguousarray(gamma, np.float32)), M, N, _p(out))
    return out


def preset_w8a8(acc, scale_token, scale_channel, bias=None):
    M, N = acc.shape
    out = np.empty((M, N), np.uint16)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().xo_preset_w8a8(_p(np.ascontiguousarray(acc, np.int32)), _p(np.ascontiguousarray(scale_token, np.float32)),
                         _p(np.ascontiguousarray(scale_channel, np.float32)), _p(b), M, N, _p(out))
    return out


def compute_rstd(x, eps=1e-6):
    x = np.ascontiguousarray(x, np.uint16)
    M, N = x.shape
    out = np.empty(M, np.float32)
    lib().xo_compute_rstd(_p(x), _p(out), M, N, C.c_float(eps))
    return out


def rstd_and_quantize(x, rstd):
    x = np.ascontiguousarray(x, np.uint16)
    M, N = x.shape
    xq = np.empty((M, N), np.int8)
    sc = np.empty(M, np.float32)
    lib().xo_rstd_and_quantize(_p(x), _p(np.ascontiguousarray(rstd, np.float32)), _p(xq), _p(sc), M, N)
    return xq, sc


def quantize_rows(x):
    x = np.ascontiguousarray(x, np.uint16)
    M, N = x.shape
    xq = np.empty((M, N), np.int8)
    sc = np.empty(M, np.float32)
    lib().xo_quantize_rows(_p(x), _p(xq), _p(sc), M, N)
    return xq, sc


def quantize_weight_cols(W):
    W = np.ascontiguousarray(W, np.uint16)
    K, N = W.shape
    Wq = np.empty((K, N), np.int8)
    sc = np.empty(N, np.float32)
    lib().xo_quantize_weight_cols(_p(W), _p(Wq), _p(sc), K, N)
    return Wq, sc


def rope_table(M, width, theta):
    cs = np.empty((M, width), np.float32)
    lib().xo_rope_table(_p(cs), M, width, C.c_float(theta))
    return cs


def quantize_columns_offline(W):
    """Offline symmetric per-column int8 quantiser, restating autotune/quantize_weights_quaRot.py:176-191:
    scale[n] = max|W[:,n]|/127 (1e-8 where that is 0); Wq = round_half_even(clip(W/scale, -128, 127)).
    Pinned by tests/golden/quantize_columns.npz, which the reference's own function produced."""
    W = np.asarray(W)
    max_abs = np.abs(W).max(axis=0, keepdims=True)
    scale = (max_abs / 127.0).squeeze(0)
    scale = np.where(scale == 0, 1e-8, scale)
    Wq = np.round(np.clip(W / scale[None, :], -128.0, 127.0)).astype(np.int8)
    return Wq, scale.astype(np.float32)


# ---- engine-style stand-alone passes (include/xe-fuse/standalone/vllm_ops.hpp) -------------------
def ve_rms_norm(x, weight, eps=1e-6):
    x = np.ascontiguousarray(x, np.uint16)
    M, N = x.shape
    out = np.empty_like(x)
    lib().xo_ve_rms_norm(_p(out), _p(x), _p(np.ascontiguousarray(weight, np.uint16)), M, N, C.c_float(eps))
    return out


def ve_fused_add_rms_norm(x, residual, weight, eps=1e-6):
    """Returns (normalised input, updated residual)."""
    x = np.array(x, np.uint16, order="C")
    r = np.array(residual, np.uint16, order="C")
    M, N = x.shape
    lib().xo_ve_fused_add_rms_norm(_p(x), _p(r), _p(np.ascontiguousarray(weight, np.uint16)), M, N,
                                   C.c_float(eps))
    return x, r


def ve_act_and_mul(x, gelu=False):
    x = np.ascontiguousarray(x, np.uint16)
    M, N2 = x.shape
    out = np.empty((M, N2 // 2), np.uint16)
    lib().xo_ve_act_and_mul(_p(out), _p(x), N2 // 2, M, 1 if gelu else 0)
    return out


def ve_rotary_neox(data, cache, head_size, rot_dim=None):
    d = np.array(data, np.uint16, order="C")
    M = d.shape[0]
    heads = d.size // (M * head_size)
    rot_dim = head_size if rot_dim is None else rot_dim
    lib().xo_ve_rotary_neox(_p(d), _p(np.ascontiguousarray(cache, np.float32)), head_size, heads, rot_dim, M)
    return d


def ve_dequant_act_mul(acc, scale_token, scale_channel, gelu=False):
    acc = np.ascontiguousarray(acc, np.int32)
    L, M, N = acc.shape if acc.ndim == 3 else (1,) + acc.shape
    out = np.empty(acc.shape, np.uint16)
    lib().xo_ve_dequant_act_mul(_p(out), _p(acc), _p(np.ascontiguousarray(scale_token, np.float32)),
                                _p(np.ascontiguousarray(scale_channel, np.float32)), N // 2, M, L,
                                1 if gelu else 0)
    return out


def ve_dequant_rotary(acc, scale_token, scale_channel, cos_sin):
    acc = np.ascontiguousarray(acc, np.int32)
    L, M, N = acc.shape if acc.ndim == 3 else (1,) + acc.shape
    out = np.empty(acc.shape, np.uint16)
    lib().xo_ve_dequant_rotary(_p(out), _p(acc), _p(np.ascontiguousarray(scale_token, np.float32)),
                               _p(np.ascontiguousarray(scale_channel, np.float32)),
                               _p(np.ascontiguousarray(cos_sin, np.float32)), M, N, L)
    return out
