"""ctypes binding of libxefuse_b200.so (the C ABI declared in include/xefuse_b200.h).

This is what the Python tests and bench.py use to drive the library; it adds nothing to the data
path.  Tensors are passed as raw device pointers (torch is only the allocator).  There is no CPU
fallback: if the shared library is missing or an entry returns an error, XfError is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libxefuse_b200.so")

# enums (include/xefuse_b200.h)
DT_BF16, DT_S8, DT_F32, DT_S32 = 0, 1, 2, 3
UNARY = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "relu": 4, "sigmoid": 5, "exp": 6}
PAIR = {"none": 0, "swiglu": 1, "geglu": 2, "rope": 3, "swap": 4}
OUT_FULL, OUT_COMPACT = 0, 1
FLAG_DIRECT_STORE, FLAG_FORCE_1CTA, FLAG_FORCE_2CTA, FLAG_FORCE_BN128, FLAG_FORCE_BN256 = 1, 2, 4, 8, 16
FLAG_FORCE_KS1, FLAG_FORCE_KS2 = 32, 64
FLAG_NO_SPLIT = 128
FLAG_NO_PDL = 4096
FLAG_SHORT_WAITS = 8192
FLAG_NO_TAIL_HELP = 32768
FLAG_NO_CLUSTER_SPLIT, FLAG_FORCE_CLUSTER_SPLIT = 65536, 131072
FLAG_NO_TAIL_STAGING = 262144
FLAG_NO_ACC_PREFETCH = 524288
FLAG_NO_RESIDUAL_TMA = 2097152
FLAG_GENERIC_EPILOGUE = 4194304
# timing diagnostics (D is garbage): honoured only with XEFUSE_ALLOW_DIAG=1 in the environment
FLAG_DIAG_NO_LOAD, FLAG_DIAG_NO_MMA, FLAG_DIAG_NO_EPILOGUE, FLAG_DIAG_NO_STORE = 256, 512, 1024, 2048
FLAG_DIAG_NO_ACC_READ = 1048576
STATIC_WORKSPACE_BYTES = 2097152

STATUS_NAMES = ["XF_SUCCESS", "XF_ERR_MISALIGNED_OPERAND", "XF_ERR_INVALID_DATA_TYPE",
                "XF_ERR_INVALID_LAYOUT", "XF_ERR_INVALID_PROBLEM", "XF_ERR_NOT_SUPPORTED",
                "XF_ERR_WORKSPACE_NULL", "XF_ERR_INTERNAL", "XF_ERR_ARCH_MISMATCH",
                "XF_ERR_INSUFFICIENT_DRIVER", "XF_ERR_MEMORY_ALLOCATION", "XF_INVALID"]


class XfError(RuntimeError):
    def __init__(self, status, text):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{name}: {text}")


class XfVec(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("enabled", C.c_int32),
                ("batch_stride", C.c_int64), ("null_default", C.c_float), ("pad_", C.c_int32)]


class XfMat(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("enabled", C.c_int32),
                ("ld", C.c_int64), ("batch_stride", C.c_int64)]


class XfEpilogueDesc(C.Structure):
    _fields_ = [("residual", XfMat), ("aux_store", XfMat), ("row_scale", XfVec),
                ("col_scale", XfVec), ("bias", XfVec), ("unary", C.c_int32), ("pair", C.c_int32),
                ("cos_sin", XfMat), ("cos_sin_period", C.c_int32), ("out_layout", C.c_int32),
                ("row_sumsq", C.c_void_p)]


class XfGemmDesc(C.Structure):
    _fields_ = [("dtype_ab", C.c_int32), ("dtype_d", C.c_int32),
                ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("L", C.c_int32),
                ("A", C.c_void_p), ("lda", C.c_int64), ("batch_a", C.c_int64),
                ("B", C.c_void_p), ("ldb", C.c_int64), ("batch_b", C.c_int64),
                ("D", C.c_void_p), ("ldd", C.c_int64), ("batch_d", C.c_int64),
                ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
                ("flags", C.c_int32), ("epi", XfEpilogueDesc),
                ("a_k_slab", C.c_int32), ("num_d_peer", C.c_int32), ("a_k_slab_stride", C.c_int64),
                ("D_peer", C.c_void_p * 7), ("workspace_bytes", C.c_uint64)]


# Every symbol include/xefuse_b200.h declares (checked by the CPU test-suite).
EXPORTS = [
    "xf_gemm_can_implement", "xf_gemm_workspace_size", "xf_gemm_plan_create", "xf_gemm_run",
    "xf_gemm_plan_device_status", "xf_gemm_plan_kernel_name", "xf_plan_destroy",
    "xf_gemm_run_static_workspace", "xf_gemm_static_workspace_status", "xf_gemm_cluster_capacity",
    "xf_last_error_string", "xf_status_string", "xf_version", "xf_compiled_arch",
    "xf_sa_scale_rows", "xf_sa_scale_cols", "xf_sa_add_residual", "xf_sa_residual_gamma",
    "xf_sa_swiglu", "xf_sa_geglu", "xf_sa_rope", "xf_sa_rope_scaled", "xf_sa_unary",
    "xf_sa_bias_add", "xf_sa_dequant_w8a8", "xf_compute_rstd", "xf_compute_rstd_and_quantize",
    "xf_row_sumsq_count", "xf_reduce_partials_rsqrt",
    "xf_ve_rms_norm", "xf_ve_fused_add_rms_norm", "xf_ve_act_and_mul", "xf_ve_rotary_embedding",
    "xf_ve_dequant_act_mul", "xf_ve_dequant_rotary",
    "xf_harness_fill_uniform", "xf_harness_ref_gemm", "xf_harness_compare",
]

_lib = None


def lib():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise XfError(7, f"{LIB_PATH} is missing: run `python xe-fuse_b200/build.py` (nvcc, sm_100a). "
                         "There is no CPU fallback.")
    L = C.CDLL(LIB_PATH)
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    L.xf_gemm_can_implement.argtypes = [C.POINTER(XfGemmDesc)]
    L.xf_gemm_workspace_size.argtypes = [C.POINTER(XfGemmDesc), C.POINTER(C.c_size_t)]
    L.xf_gemm_plan_create.argtypes = [C.POINTER(XfGemmDesc), vp, C.POINTER(vp)]
    L.xf_gemm_run.argtypes = [vp, vp]
    L.xf_gemm_plan_device_status.argtypes = [vp, C.POINTER(C.c_int32)]
    L.xf_gemm_plan_kernel_name.argtypes = [vp]
    L.xf_gemm_plan_kernel_name.restype = C.c_char_p
    L.xf_plan_destroy.argtypes = [vp]
    L.xf_gemm_run_static_workspace.argtypes = [C.POINTER(XfGemmDesc), vp]
    L.xf_gemm_static_workspace_status.argtypes = [C.POINTER(C.c_int32)]
    L.xf_gemm_cluster_capacity.argtypes = [i32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    L.xf_last_error_string.restype = C.c_char_p
    L.xf_status_string.argtypes = [i32]
    L.xf_status_string.restype = C.c_char_p
    L.xf_sa_scale_rows.argtypes = [vp, vp, i32, i32, i32, vp]
    L.xf_sa_scale_cols.argtypes = [vp, vp, i32, i32, i32, vp]
    L.xf_sa_add_residual.argtypes = [vp, vp, i32, i32, i32, vp]
    L.xf_sa_residual_gamma.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.xf_sa_swiglu.argtypes = [vp, i32, i32, i32, vp]
    L.xf_sa_geglu.argtypes = [vp, i32, i32, i32, vp]
    L.xf_sa_rope.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.xf_sa_rope_scaled.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp]
    L.xf_sa_unary.argtypes = [vp, i32, i32, i32, i32, vp]
    L.xf_sa_bias_add.argtypes = [vp, vp, i32, i32, i32, vp]
    L.xf_sa_dequant_w8a8.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp]
    L.xf_compute_rstd.argtypes = [vp, vp, i32, i32, i32, f32, vp]
    L.xf_compute_rstd_and_quantize.argtypes = [vp, vp, vp, i32, i32, i32, f32, vp]
    L.xf_row_sumsq_count.argtypes = [i32, i32, i32]
    L.xf_row_sumsq_count.restype = C.c_size_t
    L.xf_reduce_partials_rsqrt.argtypes = [vp, vp, i32, i32, i32, f32, vp]
    L.xf_ve_rms_norm.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    L.xf_ve_fused_add_rms_norm.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    L.xf_ve_act_and_mul.argtypes = [vp, vp, i32, i32, i32, vp]
    L.xf_ve_rotary_embedding.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp]
    L.xf_ve_dequant_act_mul.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp]
    L.xf_ve_dequant_rotary.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp]
    _lib = L
    return L


def check(status):
    if status != 0:
        raise XfError(status, lib().xf_last_error_string().decode())


def _torch_dtype_code(t):
    import torch
    return {torch.bfloat16: DT_BF16, torch.int8: DT_S8, torch.float32: DT_F32, torch.int32: DT_S32}[t.dtype]


def vec(t, batch_stride=0, null_default=1.0):
    """xf_vec for a 1-D torch tensor (or None => disabled)."""
    v = XfVec()
    if t is None:
        return v
    v.ptr = t.data_ptr()
    v.dtype = _torch_dtype_code(t)
    v.enabled = 1
    v.batch_stride = batch_stride
    v.null_default = null_default
    return v


def mat(t, ld=None, batch_stride=0):
    """xf_mat for a 2-D/3-D row-major torch tensor (or None => disabled)."""
    m = XfMat()
    if t is None:
        return m
    m.ptr = t.data_ptr()
    m.dtype = _torch_dtype_code(t)
    m.enabled = 1
    m.ld = ld if ld is not None else t.stride(-2)
    m.batch_stride = batch_stride if batch_stride else (t.stride(0) if t.dim() == 3 else 0)
    return m


class GemmPlan:
    """Owns an xf_plan plus the tensors it points at (keeps them alive)."""

    def __init__(self, A, B, D, *, residual=None, aux_store=None, row_scale=None, col_scale=None,
                 bias=None, unary="none", pair="none", cos_sin=None, cos_sin_period=0,
                 compact=False, flags=0, tile=(256, 256, 32), a_k_slabs=False, d_peer_ptrs=(),
                 row_sumsq=None):
        import torch
        L_ = lib()
        self._keep = [A, B, D, residual, aux_store, row_scale, col_scale, bias, cos_sin, row_sumsq]
        batched = A.dim() == 3 and not a_k_slabs
        Lb = A.shape[0] if batched else 1
        M, K = A.shape[-2], A.shape[-1]
        if a_k_slabs:          # A is [G][M, K/G]: the gathered output of G column shards
            K = A.shape[0] * A.shape[2]
        N = B.shape[-1]
        d = XfGemmDesc()
        d.dtype_ab = _torch_dtype_code(A)
        d.dtype_d = _torch_dtype_code(D)
        d.M, d.N, d.K, d.L = M, N, K, Lb
        d.A, d.lda, d.batch_a = A.data_ptr(), A.stride(-2), (A.stride(0) if batched else 0)
        bb = B.dim() == 3
        d.B, d.ldb, d.batch_b = B.data_ptr(), B.stride(-2), (B.stride(0) if bb else 0)
        d.D, d.ldd, d.batch_d = D.data_ptr(), D.stride(-2), (D.stride(0) if D.dim() == 3 else 0)
        d.tile_m, d.tile_n, d.tile_k = tile
        d.flags = flags
        if a_k_slabs:
            d.a_k_slab, d.a_k_slab_stride = A.shape[2], A.stride(0)
        d.num_d_peer = len(d_peer_ptrs)        # raw device pointers of further copies of D
        for i, ptr in enumerate(d_peer_ptrs):
            d.D_peer[i] = ptr
        e = d.epi
        e.residual = mat(residual)
        e.aux_store = mat(aux_store)
        e.row_scale = vec(row_scale, batch_stride=M)
        e.col_scale = vec(col_scale, batch_stride=N)
        e.bias = vec(bias, batch_stride=N, null_default=0.0)
        e.unary = UNARY[unary]
        e.pair = PAIR[pair]
        e.cos_sin = mat(cos_sin)
        e.cos_sin_period = cos_sin_period
        e.out_layout = OUT_COMPACT if compact else OUT_FULL
        e.row_sumsq = row_sumsq.data_ptr() if row_sumsq is not None else None
        self.desc = d
        check(L_.xf_gemm_can_implement(C.byref(d)))
        ws = C.c_size_t(0)
        check(L_.xf_gemm_workspace_size(C.byref(d), C.byref(ws)))
        self.workspace = torch.zeros(max(int(ws.value), 16), dtype=torch.uint8, device=A.device)
        d.workspace_bytes = self.workspace.numel()
        self.handle = C.c_void_p()
        check(L_.xf_gemm_plan_create(C.byref(d), self.workspace.data_ptr(), C.byref(self.handle)))
        self.kernel_name = L_.xf_gemm_plan_kernel_name(self.handle).decode()
        self.flops = 2.0 * M * N * K * Lb

    def run(self, stream=None):
        import torch
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(lib().xf_gemm_run(self.handle, s))

    def device_status(self):
        code = C.c_int32(0)
        check(lib().xf_gemm_plan_device_status(self.handle, C.byref(code)))
        return code.value

    def close(self):
        if self.handle:
            lib().xf_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def cluster_capacity(dtype_code=DT_BF16):
    """(CTA pairs, 4-CTA clusters) the current device holds at once: the planner's scheduling units."""
    pairs, quads = C.c_int32(0), C.c_int32(0)
    check(lib().xf_gemm_cluster_capacity(dtype_code, C.byref(pairs), C.byref(quads)))
    return pairs.value, quads.value


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def sa_scale_rows(D, scale):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_scale_rows(D.data_ptr(), scale.data_ptr(), M, N, L_, _stream()))


def sa_scale_cols(D, scale):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_scale_cols(D.data_ptr(), scale.data_ptr(), M, N, L_, _stream()))


def sa_add_residual(D, residual):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_add_residual(D.data_ptr(), residual.data_ptr(), M, N, L_, _stream()))


def sa_residual_gamma(D, residual, gamma):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_residual_gamma(D.data_ptr(), residual.data_ptr(), gamma.data_ptr(), M, N, L_, _stream()))


def sa_swiglu(D):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_swiglu(D.data_ptr(), M, N, L_, _stream()))


def sa_geglu(D):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_geglu(D.data_ptr(), M, N, L_, _stream()))


def sa_rope(out, inp, cos_sin):
    L_, M, N = _lmn(out)
    check(lib().xf_sa_rope(out.data_ptr(), inp.data_ptr(), cos_sin.data_ptr(), M, N, L_, _stream()))


def sa_rope_scaled(out, inp, scale, cos_sin):
    L_, M, N = _lmn(out)
    check(lib().xf_sa_rope_scaled(out.data_ptr(), inp.data_ptr(), scale.data_ptr(), cos_sin.data_ptr(),
                                  M, N, L_, _stream()))


def sa_unary(D, name):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_unary(D.data_ptr(), UNARY[name], M, N, L_, _stream()))


def sa_bias_add(D, bias):
    L_, M, N = _lmn(D)
    check(lib().xf_sa_bias_add(D.data_ptr(), bias.data_ptr(), M, N, L_, _stream()))


def sa_dequant_w8a8(out, acc, scale_token, scale_channel):
    L_, M, N = _lmn(out)
    check(lib().xf_sa_dequant_w8a8(out.data_ptr(), acc.data_ptr(), scale_token.data_ptr(),
                                   scale_channel.data_ptr(), M, N, L_, _stream()))


def compute_rstd(x, rstd, eps=1e-6):
    L_, M, N = _lmn(x)
    check(lib().xf_compute_rstd(x.data_ptr(), rstd.data_ptr(), M, N, L_, eps, _stream()))


def compute_rstd_and_quantize(x, xq, scale_token, eps=1e-6):
    L_, M, N = _lmn(x)
    check(lib().xf_compute_rstd_and_quantize(x.data_ptr(), xq.data_ptr(), scale_token.data_ptr(),
                                             M, N, L_, eps, _stream()))


def _lmn(t):
    if not t.is_contiguous():
        raise XfError(3, "stand-alone ops take packed row-major tensors")
    if t.dim() == 3:
        return t.shape[0], t.shape[1], t.shape[2]
    return 1, t.shape[0], t.shape[1]


# ---- engine-style row passes (xf_ve_*): the comparison arm of the reference's pipelines ----------
def ve_rms_norm(out, inp, weight, eps=1e-6):
    M, N = inp.shape
    check(lib().xf_ve_rms_norm(out.data_ptr(), inp.data_ptr(), weight.data_ptr(), M, N, eps, _stream()))


def ve_fused_add_rms_norm(inp, residual, weight, eps=1e-6):
    M, N = inp.shape
    check(lib().xf_ve_fused_add_rms_norm(inp.data_ptr(), residual.data_ptr(), weight.data_ptr(), M, N, eps,
                                         _stream()))


def ve_act_and_mul(out, inp, gelu=False):
    M, d = out.shape
    check(lib().xf_ve_act_and_mul(out.data_ptr(), inp.data_ptr(), d, M, 1 if gelu else 0, _stream()))


def ve_rotary_embedding(query, key, cos_sin_cache, head_size, rot_dim=None):
    M = query.shape[0]
    rot_dim = head_size if rot_dim is None else rot_dim
    nq = query.numel() // (M * head_size)
    nk = key.numel() // (M * head_size) if key is not None else 0
    check(lib().xf_ve_rotary_embedding(query.data_ptr(), key.data_ptr() if key is not None else None,
                                       cos_sin_cache.data_ptr(), head_size, nq, nk, rot_dim, M, _stream()))


def ve_dequant_act_mul(out, acc, scale_token, scale_channel, gelu=False):
    L_, M, N = _lmn(out)
    check(lib().xf_ve_dequant_act_mul(out.data_ptr(), acc.data_ptr(), scale_token.data_ptr(),
                                      scale_channel.data_ptr(), N // 2, M, L_, 1 if gelu else 0, _stream()))


def ve_dequant_rotary(out, acc, scale_token, scale_channel, cos_sin):
    L_, M, N = _lmn(out)
    check(lib().xf_ve_dequant_rotary(out.data_ptr(), acc.data_ptr(), scale_token.data_ptr(),
                                     scale_channel.data_ptr(), cos_sin.data_ptr(), M, N, L_, _stream()))


def reduce_partials_rsqrt(partials, rstd, M, N, L=1, eps=1e-6):
    """rstd from the row_sumsq side output of a fused GEMM."""
    check(lib().xf_reduce_partials_rsqrt(partials.data_ptr(), rstd.data_ptr(), M, N, L, eps, _stream()))
