"""Seeded inputs and expected outputs for the fused-GEMM presets.

Each case names a preset of the reference's kernel generator (autotune/generate_kernel.py:50-407),
builds its inputs on the host from a fixed seed, and gives (a) the keyword arguments of the flat
epilogue for the GPU path and (b) the oracle's expected output.  Used by the GPU parity tests, the
smoke check and the golden fixtures.
"""
import numpy as np

# Parity bar for bf16 outputs against the fp32 host reference: an element passes when its absolute
# error is <= ATOL or its relative error is <= RTOL.
ATOL = 2e-2
RTOL = 1e-2

PRESETS = ["k1", "k1v2", "k2", "k2_compact", "k2_geglu", "k2v2", "k3", "k4", "k4v2", "k4v2_table",
           "k0a", "k0_dual", "w8a8_dequant", "w8a8_dequant_biased", "w8a8_biased_bf16bias",
           "bias_gelu", "bias_gelu_tanh", "scale_silu", "relu", "sigmoid", "w8a8_rope", "w8a8_swiglu",
           "w8a8_geglu", "identity"]


def is_int8(preset):
    return preset.startswith("w8a8")


def make_inputs(o, preset, M, N, K, seed=0):
    """Returns a dict of numpy arrays (bf16 as uint16 bits)."""
    rng = np.random.default_rng(seed + 1000 * (sum(map(ord, preset)) % 97))
    d = {}
    if is_int8(preset):
        x = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        w = o.f32_to_bf16((rng.standard_normal((K, N)) * K ** -0.5).astype(np.float32))
        d["A"], d["scale_token"] = o.quantize_rows(x)          # per-token absmax symmetric
        d["B"], d["scale_channel"] = o.quantize_weight_cols(w)  # per-channel absmax
    else:
        d["A"] = o.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        d["B"] = o.f32_to_bf16((rng.standard_normal((K, N)) * K ** -0.5).astype(np.float32))
        d["scale"] = o.compute_rstd(d["A"], 1e-6)               # R[m] = rsqrt(mean(x^2)+1e-6)
    d["gamma"] = rng.normal(1.0, 0.02, N).astype(np.float32)
    d["bias"] = rng.normal(0.0, 0.02, N).astype(np.float32)
    d["bias_bf16"] = o.f32_to_bf16(d["bias"])
    d["residual"] = o.f32_to_bf16(rng.standard_normal((M, N)).astype(np.float32))
    d["cos_sin_full"] = o.rope_table(M, N, 10000.0) if N % 2 == 0 else None   # reference form
    P = 128 if N % 128 == 0 else (32 if N % 32 == 0 else 0)
    d["period"] = P
    d["cos_sin_table"] = o.rope_table(M, P, 500000.0) if P else None           # per-head table
    return d


def epilogue_kwargs(o, preset, d):
    """(kwargs for oracle.epilogue / the GPU plan, compact flag)."""
    k = {}
    if preset in ("k1", "k1v2"):
        k = dict(row=d["scale"])
    elif preset in ("k2", "k2v2"):
        k = dict(row=d["scale"], pair="swiglu")
    elif preset == "k2_compact":
        k = dict(row=d["scale"], pair="swiglu", compact=True)
    elif preset == "k2_geglu":
        k = dict(row=d["scale"], pair="geglu")
    elif preset == "k3":
        k = dict(pair="rope", cos_sin=d["cos_sin_full"])
    elif preset in ("k4", "k4v2"):
        k = dict(row=d["scale"], pair="rope", cos_sin=d["cos_sin_full"])
    elif preset == "k4v2_table":
        k = dict(row=d["scale"], pair="rope", cos_sin=d["cos_sin_table"], cos_sin_period=d["period"])
    elif preset == "k0a":
        k = dict(residual=d["residual"], col=d["gamma"])
    elif preset == "k0_dual":
        k = dict(residual=d["residual"], col=d["gamma"], want_aux=True)
    elif preset == "w8a8_dequant":
        k = dict(row=d["scale_token"], col=d["scale_channel"])
    elif preset == "w8a8_dequant_biased":
        k = dict(row=d["scale_token"], col=d["scale_channel"], bias=d["bias"])
    elif preset == "w8a8_biased_bf16bias":
        k = dict(row=d["scale_token"], col=d["scale_channel"], bias=o.bf16_to_f32(d["bias_bf16"]))
    elif preset == "w8a8_rope":
        k = dict(row=d["scale_token"], col=d["scale_channel"], pair="rope", cos_sin=d["cos_sin_full"])
    elif preset == "w8a8_swiglu":
        k = dict(row=d["scale_token"], col=d["scale_channel"], pair="swiglu")
    elif preset == "w8a8_geglu":      # DequantGeGLU, builder/epilogue_builder.hpp:276-280
        k = dict(row=d["scale_token"], col=d["scale_channel"], pair="geglu")
    elif preset == "bias_gelu":
        k = dict(bias=d["bias"], unary="gelu")
    elif preset == "bias_gelu_tanh":
        k = dict(bias=d["bias"], unary="gelu_tanh")
    elif preset == "scale_silu":
        k = dict(row=d["scale"], unary="silu")
    elif preset == "relu":
        k = dict(unary="relu")
    elif preset == "sigmoid":
        k = dict(unary="sigmoid")
    elif preset == "identity":
        k = {}
    else:
        raise KeyError(preset)
    return k


def expected(o, preset, d):
    """Oracle result: (accumulator, bf16 output bits[, aux bits])."""
    acc = o.gemm_s8(d["A"], d["B"]) if is_int8(preset) else o.gemm_bf16(d["A"], d["B"])
    out = o.epilogue(acc, **epilogue_kwargs(o, preset, d))
    return acc, out


def compare_bf16(o, got_bits, want_bits):
    """Returns (n_bad, max_abs_err, max_rel_err) under the ATOL-or-RTOL bar."""
    g = o.bf16_to_f32(got_bits).astype(np.float64)
    w = o.bf16_to_f32(want_bits).astype(np.float64)
    err = np.abs(g - w)
    rel = err / np.maximum(np.abs(w), 1e-30)
    bad = ~((err <= ATOL) | (rel <= RTOL)) | ~np.isfinite(g)
    return int(bad.sum()), float(err.max()) if err.size else 0.0, float(rel[np.abs(w) > 1e-3].max()) if (np.abs(w) > 1e-3).any() else 0.0
