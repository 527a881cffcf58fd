// Scalar and small-vector arithmetic shared by every Field kernel.
//
// Everything here is a plain inline function of its arguments, marked for host
// and device, so that the same source can be compiled by nvcc for sm_100a and
// by g++ for the host-side kernel emulation used by the CPU tests
// (FIELDS_HOST_EMU).
//
// Reference arithmetic being reproduced (file field_only_v4_chunked_triton_wiki100.py):
//   gates          :493-501   inj = tanh(z_r) + i tanh(z_i), v = 0.9 sigmoid(z_v)
//   coefficients   :497-501   a = (1 - v) lambda, b = gamma v inj
//   compose        :503-509   (A, B) <- (a A, a B + b)
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

#ifdef FIELDS_HOST_EMU
#define FL_HD inline
#define FL_DEVICE_CODE 0
#else
#include <cuda_runtime.h>
#define FL_HD __host__ __device__ __forceinline__
#ifdef __CUDA_ARCH__
#define FL_DEVICE_CODE 1
#else
#define FL_DEVICE_CODE 0
#endif
#endif

namespace fields {

constexpr float kVacMax = 0.90f;  // VAC_MAX, field_only_v4_chunked_triton_wiki100.py:68

// ---------------------------------------------------------------------------
// Transcendentals: one ex2.approx and one rcp.approx each (about 2 ulp), which the
// recurrence carries to well under the 1e-5 parity bound. No clamping is needed: the
// hardware returns +inf / +0 for large arguments of ex2 and +0 for rcp(+inf), so tanh
// saturates to +-1 and sigmoid to 0 or 1; the host forms below do the same in IEEE
// arithmetic.
//   tanh(x)    = 1 - 2 / (2^(2 log2e x) + 1)
//   sigmoid(x) = 1 / (1 + 2^(-log2e x))
// ---------------------------------------------------------------------------
constexpr float kLog2e = 1.4426950408889634f;

FL_HD float fast_exp2(float x) {
#if FL_DEVICE_CODE
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
#else
    return std::exp2(x);
#endif
}

FL_HD float fast_rcp(float x) {
#if FL_DEVICE_CODE
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
#else
    return 1.0f / x;
#endif
}

FL_HD float sigmoidf_fast(float x) { return fast_rcp(1.0f + fast_exp2(-kLog2e * x)); }

FL_HD float tanhf_fast(float x) {
    return 1.0f - 2.0f * fast_rcp(fast_exp2((2.0f * kLog2e) * x) + 1.0f);
}

// ---------------------------------------------------------------------------
// Vec<V>: V consecutive channels held by one thread. V = 4 moves 128 bits per
// access and needs 16-byte aligned addresses; V = 1 is the fallback for channel
// counts that are not a multiple of four.
// ---------------------------------------------------------------------------
template <int V>
struct Vec {
    float v[V];
};

template <int V>
FL_HD Vec<V> vec_fill(float x) {
    Vec<V> r;
#pragma unroll
    for (int k = 0; k < V; ++k) r.v[k] = x;
    return r;
}

// Ordinary load (data that is read again soon: stays in L2).
template <int V>
FL_HD Vec<V> vec_load(const float* p) {
    Vec<V> r;
#if FL_DEVICE_CODE
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else if constexpr (V == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        r.v[0] = t.x; r.v[1] = t.y;
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) r.v[k] = p[k];
    }
#else
    std::memcpy(r.v, p, sizeof(float) * V);
#endif
    return r;
}

// Streaming load (data read once: evict first).
template <int V>
FL_HD Vec<V> vec_load_stream(const float* p) {
    Vec<V> r;
#if FL_DEVICE_CODE
    if constexpr (V == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else if constexpr (V == 2) {
        const float2 t = __ldcs(reinterpret_cast<const float2*>(p));
        r.v[0] = t.x; r.v[1] = t.y;
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) r.v[k] = __ldcs(p + k);
    }
#else
    std::memcpy(r.v, p, sizeof(float) * V);
#endif
    return r;
}

// Load cached in L2 only (data that another pass reads again, no use for L1).
template <int V>
FL_HD Vec<V> vec_load_l2(const float* p) {
    Vec<V> r;
#if FL_DEVICE_CODE
    if constexpr (V == 4) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) r.v[k] = __ldcg(p + k);
    }
#else
    std::memcpy(r.v, p, sizeof(float) * V);
#endif
    return r;
}

template <int V>
FL_HD void vec_store(float* p, const Vec<V>& x) {
#if FL_DEVICE_CODE
    if constexpr (V == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
    } else if constexpr (V == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(x.v[0], x.v[1]);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) p[k] = x.v[k];
    }
#else
    std::memcpy(p, x.v, sizeof(float) * V);
#endif
}

// Streaming store (output that this kernel never reads back).
template <int V>
FL_HD void vec_store_stream(float* p, const Vec<V>& x) {
#if FL_DEVICE_CODE
    if constexpr (V == 4) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(x.v[0], x.v[1], x.v[2], x.v[3]));
    } else if constexpr (V == 2) {
        __stcs(reinterpret_cast<float2*>(p), make_float2(x.v[0], x.v[1]));
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) __stcs(p + k, x.v[k]);
    }
#else
    std::memcpy(p, x.v, sizeof(float) * V);
#endif
}

// ---------------------------------------------------------------------------
// bfloat16 as raw bits (uint16_t): conversions that work on host and device alike, and
// 4-element vector I/O for both element types (float: 16 bytes, bf16: 8 bytes per access).
// ---------------------------------------------------------------------------
FL_HD float bf16_bits_to_float(uint16_t h) {
    const uint32_t u = (uint32_t)h << 16;
    float f;
#if FL_DEVICE_CODE
    f = __uint_as_float(u);
#else
    std::memcpy(&f, &u, 4);
#endif
    return f;
}

// round to nearest even; NaN stays NaN
FL_HD uint16_t float_to_bf16_bits(float f) {
    uint32_t u;
#if FL_DEVICE_CODE
    u = __float_as_uint(f);
#else
    std::memcpy(&u, &f, 4);
#endif
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}


FL_HD Vec<4> io_load4(const float* p) { return vec_load<4>(p); }
FL_HD Vec<4> io_load4_stream(const float* p) { return vec_load_stream<4>(p); }
FL_HD void io_store4_stream(float* p, const Vec<4>& x) { vec_store_stream<4>(p, x); }

FL_HD Vec<4> bf16x4_unpack(uint32_t lo, uint32_t hi) {
    Vec<4> r;
    r.v[0] = bf16_bits_to_float((uint16_t)(lo & 0xffffu));
    r.v[1] = bf16_bits_to_float((uint16_t)(lo >> 16));
    r.v[2] = bf16_bits_to_float((uint16_t)(hi & 0xffffu));
    r.v[3] = bf16_bits_to_float((uint16_t)(hi >> 16));
    return r;
}

FL_HD Vec<4> io_load4(const uint16_t* p) {
#if FL_DEVICE_CODE
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    return bf16x4_unpack(t.x, t.y);
#else
    uint32_t w[2];
    std::memcpy(w, p, 8);
    return bf16x4_unpack(w[0], w[1]);
#endif
}

FL_HD Vec<4> io_load4_stream(const uint16_t* p) {
#if FL_DEVICE_CODE
    const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    return bf16x4_unpack(t.x, t.y);
#else
    return io_load4(p);
#endif
}

FL_HD void io_store4_stream(uint16_t* p, const Vec<4>& x) {
#if FL_DEVICE_CODE
    // one conversion instruction per pair (round to nearest even; the upper half is the first operand)
    uint32_t lo, hi;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(x.v[1]), "f"(x.v[0]));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x.v[3]), "f"(x.v[2]));
    __stcs(reinterpret_cast<uint2*>(p), make_uint2(lo, hi));
#else
    const uint32_t lo = (uint32_t)float_to_bf16_bits(x.v[0]) | ((uint32_t)float_to_bf16_bits(x.v[1]) << 16);
    const uint32_t hi = (uint32_t)float_to_bf16_bits(x.v[2]) | ((uint32_t)float_to_bf16_bits(x.v[3]) << 16);
    const uint32_t w[2] = {lo, hi};
    std::memcpy(p, w, 8);
#endif
}

// ---------------------------------------------------------------------------
// F2: two adjacent channels in one 64-bit register pair. On sm_100 add, multiply and
// fused multiply-add exist in a packed form that executes both lanes with one
// instruction (fma.rn.f32x2 and friends), which halves the issue slots the complex
// arithmetic needs; the hot loops are issue-limited at the occupancy their registers allow.
// Each lane is an ordinary IEEE fp32 operation. The host forms do the same per lane.
// ---------------------------------------------------------------------------
struct alignas(8) F2 {
    float x, y;
};

FL_HD F2 splat2(float s) { return F2{s, s}; }
FL_HD F2 lo2(const Vec<4>& v) { return F2{v.v[0], v.v[1]}; }
FL_HD F2 hi2(const Vec<4>& v) { return F2{v.v[2], v.v[3]}; }
FL_HD Vec<4> join2(const F2& a, const F2& b) {
    Vec<4> r;
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y;
    return r;
}

// a * b + c
FL_HD F2 fma2(const F2& a, const F2& b, const F2& c) {
#if FL_DEVICE_CODE
    const float2 r = __ffma2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y), make_float2(c.x, c.y));
    return F2{r.x, r.y};
#else
    return F2{a.x * b.x + c.x, a.y * b.y + c.y};
#endif
}

FL_HD F2 mul2(const F2& a, const F2& b) {
#if FL_DEVICE_CODE
    const float2 r = __fmul2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y));
    return F2{r.x, r.y};
#else
    return F2{a.x * b.x, a.y * b.y};
#endif
}

FL_HD F2 add2(const F2& a, const F2& b) {
#if FL_DEVICE_CODE
    const float2 r = __fadd2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y));
    return F2{r.x, r.y};
#else
    return F2{a.x + b.x, a.y + b.y};
#endif
}

FL_HD F2 exp2_2(const F2& a) { return F2{fast_exp2(a.x), fast_exp2(a.y)}; }
FL_HD F2 rcp2(const F2& a) { return F2{fast_rcp(a.x), fast_rcp(a.y)}; }

// Gates of two channels. `rr`, `ri` are the reciprocals inside the tanh form
// (tanh = 1 - 2 r), kept because 1 - tanh^2 = (1 - 2 r)(2 r - 1) + 1 needs them.
struct Gate2 {
    F2 inj_r, inj_i, rr, ri, sig, vac, keep;
};

FL_HD F2 sigmoid2(const F2& z) {
    return rcp2(add2(exp2_2(mul2(z, splat2(-kLog2e))), splat2(1.0f)));
}

FL_HD Gate2 make_gate2(const F2& zr, const F2& zi, const F2& zv) {
    Gate2 g;
    const F2 one = splat2(1.0f), k2 = splat2(2.0f * kLog2e), m2 = splat2(-2.0f);
    g.rr = rcp2(add2(exp2_2(mul2(zr, k2)), one));
    g.ri = rcp2(add2(exp2_2(mul2(zi, k2)), one));
    g.inj_r = fma2(g.rr, m2, one);
    g.inj_i = fma2(g.ri, m2, one);
    g.sig = sigmoid2(zv);
    g.vac = mul2(g.sig, splat2(kVacMax));
    g.keep = fma2(g.sig, splat2(-kVacMax), one);
    return g;
}

// Affine maps of two channels.
struct Affine2 {
    F2 ar, ai, br, bi;
};

FL_HD Affine2 affine2_identity() {
    return Affine2{splat2(1.0f), splat2(0.0f), splat2(0.0f), splat2(0.0f)};
}

// ---------------------------------------------------------------------------
// Per-channel gate values of one time step.
// ---------------------------------------------------------------------------
struct Gate {
    float inj_r, inj_i;  // tanh(z_r), tanh(z_i)
    float sig;           // sigmoid(z_v)
    float vac;           // 0.9 * sig
};

FL_HD Gate make_gate(float zr, float zi, float zv) {
    Gate g;
    g.inj_r = tanhf_fast(zr);
    g.inj_i = tanhf_fast(zi);
    g.sig = sigmoidf_fast(zv);
    g.vac = kVacMax * g.sig;
    return g;
}

// Complex helpers on (re, im) pairs.
FL_HD void cmul(float ar, float ai, float br, float bi, float& or_, float& oi) {
    or_ = ar * br - ai * bi;
    oi = ar * bi + ai * br;
}
// conj(a) * b
FL_HD void cmul_conj(float ar, float ai, float br, float bi, float& or_, float& oi) {
    or_ = ar * br + ai * bi;
    oi = ar * bi - ai * br;
}

// Affine map s -> A s + B on one complex channel.
struct Affine {
    float ar, ai, br, bi;
};

FL_HD Affine affine_identity() { return Affine{1.0f, 0.0f, 0.0f, 0.0f}; }

// The map "first m, then step (a, b)":  s -> a (A s + B) + b.
FL_HD Affine affine_then(const Affine& m, float a_r, float a_i, float b_r, float b_i) {
    Affine o;
    o.br = a_r * m.br - a_i * m.bi + b_r;
    o.bi = a_r * m.bi + a_i * m.br + b_i;
    o.ar = a_r * m.ar - a_i * m.ai;
    o.ai = a_r * m.ai + a_i * m.ar;
    return o;
}

FL_HD void affine_apply(const Affine& m, float& sr, float& si) {
    const float nr = m.ar * sr - m.ai * si + m.br;
    const float ni = m.ar * si + m.ai * sr + m.bi;
    sr = nr;
    si = ni;
}

}  // namespace fields
