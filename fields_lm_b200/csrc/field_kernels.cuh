// Chunk-parallel kernels for the Field recurrence (three launches per direction).
//
// Time is cut into chunks of `ts` steps. One warp owns one (batch, chunk,
// channel-group) tile; a lane owns VEC consecutive channels, so a warp reads and
// writes 32*VEC consecutive floats of one plane of one time step per access
// (512 contiguous bytes with VEC = 4: 128-bit accesses, fully coalesced).
//
//   forward   FwdSummary      chunk -> affine map (A, B)        reads raw once
//             FwdCarry        exclusive scan of the maps        workspace only
//             FwdMaterialize  recurrence from the carry, writes read
//   backward  BwdSummary      chunk -> dual map (P, Q)          reads z_v, grad_read
//             BwdCarry        reverse exclusive scan
//             BwdMaterialize  reverse recurrence, writes grad_raw and partials
//             BwdReduce       fixed-order sum of the partials -> [C]
//
// The same decomposition as the reference's six Triton kernels
// (field_only_v4_chunked_triton_wiki100.py:443-909) but with a different
// mapping: 128-bit lanes over channels, unrolled loads running ahead of the
// serial dependency, a two-level carry scan instead of a serial one, and a
// deterministic in-library reduction of the parameter gradients.
//
// Every kernel is a struct with `phaseN(params, block, thread, smem)` bodies.
// Phases are separated by a block barrier and communicate only through shared
// or global memory, which lets the CPU tests run the very same bodies in nested
// loops (FIELDS_HOST_EMU) to check index arithmetic and formulas without a GPU.
#pragma once

#include "field_math.cuh"

namespace fields {

struct Shape {
    int B, L, C;
    int ts;  // time steps per chunk
    int N;   // chunks per sequence = ceil(L / ts)
    int G;   // channel groups per row = ceil(C / (32 * VEC))
};

struct FwdParams {
    const float* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;  // [B, 2C] or null
    float* read;            // [B, L, 4C]
    float* state_out;       // [B, 2C] or null
    float* sum;             // [4][B][N][C]  Re A | Im A | Re B | Im B
    float* carry;           // [2][B][N][C]  state entering each chunk
    Shape s;
};

struct BwdParams {
    const float* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;        // [B, 2C] or null
    const float* read;            // saved forward output [B, L, 4C]
    const float* grad_read;       // [B, L, 4C]
    const float* grad_state_out;  // [B, 2C] or null
    float* grad_raw;              // [B, L, 3C]
    float* grad_state_in;         // [B, 2C] or null
    float* sum;                   // [4][B][N][C]  Re P | Im P | Re Q | Im Q
    float* carry;                 // [2][B][N][C]  gradient carry entering each chunk from later time
    float* partial;               // [3][B][N][C]  d lambda_r | d lambda_i | d gamma
    float* grad_tr;
    float* grad_ti;
    float* grad_gamma;
    Shape s;
};

constexpr int kWarpsPerBlock = 4;  // tile kernels: 4 warps = one full 512-channel row with VEC = 4

struct Tile {
    int b, n, c0;
    int tbeg, tend;
    bool active;
};

template <int VEC>
FL_HD Tile decode_tile(const Shape& s, int block, int thread) {
    Tile t;
    const int lane = thread & 31;
    const long long task = (long long)block * kWarpsPerBlock + (thread >> 5);
    const long long total = (long long)s.B * s.N * s.G;
    const int cg = (int)(task % s.G);
    t.n = (int)((task / s.G) % s.N);
    t.b = (int)(task / ((long long)s.G * s.N));
    t.c0 = (cg * 32 + lane) * VEC;
    t.tbeg = t.n * s.ts;
    t.tend = t.tbeg + s.ts < s.L ? t.tbeg + s.ts : s.L;
    t.active = task < total && t.c0 < s.C;
    return t;
}

// ---------------------------------------------------------------------------
// Forward 1/3: affine summary of every chunk.
// ---------------------------------------------------------------------------
template <int VEC, int U>
struct FwdSummary {
    using Params = FwdParams;
    static constexpr int kThreads = 32 * kWarpsPerBlock;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const Shape& s = p.s;
        const Tile tl = decode_tile<VEC>(s, block, thread);
        if (!tl.active) return;
        const int C = s.C;
        const Vec<VEC> lr = vec_load<VEC>(p.tr + tl.c0);
        const Vec<VEC> li = vec_load<VEC>(p.ti + tl.c0);
        const Vec<VEC> gm = vec_load<VEC>(p.gamma + tl.c0);
        Affine m[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) m[k] = affine_identity();

        const float* base = p.raw + (size_t)tl.b * s.L * 3 * C + tl.c0;
        for (int t0 = tl.tbeg; t0 < tl.tend; t0 += U) {
            Vec<VEC> zr[U], zi[U], zv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 + u < tl.tend) {
                    const float* row = base + (size_t)(t0 + u) * 3 * C;
                    zr[u] = vec_load<VEC>(row);
                    zi[u] = vec_load<VEC>(row + C);
                    zv[u] = vec_load<VEC>(row + 2 * C);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 + u < tl.tend) {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const Gate g = make_gate(zr[u].v[k], zi[u].v[k], zv[u].v[k]);
                        const float keep = 1.0f - g.vac;
                        const float bs = gm.v[k] * g.vac;
                        m[k] = affine_then(m[k], keep * lr.v[k], keep * li.v[k],
                                           bs * g.inj_r, bs * g.inj_i);
                    }
                }
            }
        }
        const size_t plane = (size_t)s.B * s.N * C;
        float* out = p.sum + ((size_t)tl.b * s.N + tl.n) * C + tl.c0;
        Vec<VEC> o0, o1, o2, o3;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            o0.v[k] = m[k].ar; o1.v[k] = m[k].ai; o2.v[k] = m[k].br; o3.v[k] = m[k].bi;
        }
        vec_store<VEC>(out, o0);
        vec_store<VEC>(out + plane, o1);
        vec_store<VEC>(out + 2 * plane, o2);
        vec_store<VEC>(out + 3 * plane, o3);
    }
};

// ---------------------------------------------------------------------------
// Forward 2/3 and backward 2/3: exclusive scan of the chunk maps, two levels.
// One block owns 32 channels of one batch row; warp w composes the chunks of
// its slice (phase 0, result to shared memory), then every warp folds the
// slices before it into its incoming state and walks its slice again writing
// the state that enters each chunk (phase 1).
//   REVERSE = false: chunks ascending, start = state_in       (forward)
//   REVERSE = true : chunks descending, start = grad_state_out (backward);
//                    the value left after chunk 0 is grad_state_in.
// ---------------------------------------------------------------------------
constexpr int kCarryWarps = 16;

template <bool REVERSE>
struct CarryScan {
    struct Params {
        const float* sum;    // [4][B][N][C]
        float* carry;        // [2][B][N][C]
        const float* start;  // [B, 2C] or null
        float* finish;       // [B, 2C] or null: state after the last chunk in scan order
        Shape s;
    };
    static constexpr int kThreads = 32 * kCarryWarps;
    static constexpr int kPhases = 2;
    static constexpr int kSmemFloats = 4 * kThreads;

    struct Slice {
        int b, c, lo, hi, w, lane;  // chunks [lo, hi) in scan order index
        bool active;
    };

    FL_HD static Slice decode(const Shape& s, int block, int thread) {
        Slice sl;
        const int cgroups = (s.C + 31) / 32;
        sl.lane = thread & 31;
        sl.w = thread >> 5;
        sl.b = block / cgroups;
        sl.c = (block % cgroups) * 32 + sl.lane;
        const int per = (s.N + kCarryWarps - 1) / kCarryWarps;
        sl.lo = sl.w * per < s.N ? sl.w * per : s.N;
        sl.hi = sl.lo + per < s.N ? sl.lo + per : s.N;
        sl.active = sl.c < s.C && sl.b < s.B;
        return sl;
    }

    // scan-order index -> chunk number
    FL_HD static int chunk_of(const Shape& s, int i) { return REVERSE ? s.N - 1 - i : i; }

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const Slice sl = decode(s, block, thread);
        if (!sl.active) return;
        const size_t plane = (size_t)s.B * s.N * s.C;
        Affine m = affine_identity();
        for (int i = sl.lo; i < sl.hi; ++i) {
            const size_t idx = ((size_t)sl.b * s.N + chunk_of(s, i)) * s.C + sl.c;
            m = affine_then(m, p.sum[idx], p.sum[idx + plane], p.sum[idx + 2 * plane],
                            p.sum[idx + 3 * plane]);
        }
        float* o = smem + 4 * thread;
        o[0] = m.ar; o[1] = m.ai; o[2] = m.br; o[3] = m.bi;
    }

    FL_HD static void phase1(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const Slice sl = decode(s, block, thread);
        if (!sl.active) return;
        const size_t plane = (size_t)s.B * s.N * s.C;
        float sr = p.start ? p.start[(size_t)sl.b * 2 * s.C + sl.c] : 0.0f;
        float si = p.start ? p.start[(size_t)sl.b * 2 * s.C + s.C + sl.c] : 0.0f;
        for (int w = 0; w < sl.w; ++w) {
            const float* q = smem + 4 * (w * 32 + sl.lane);
            affine_apply(Affine{q[0], q[1], q[2], q[3]}, sr, si);
        }
        for (int i = sl.lo; i < sl.hi; ++i) {
            const size_t idx = ((size_t)sl.b * s.N + chunk_of(s, i)) * s.C + sl.c;
            p.carry[idx] = sr;
            p.carry[idx + plane] = si;
            affine_apply(Affine{p.sum[idx], p.sum[idx + plane], p.sum[idx + 2 * plane],
                                p.sum[idx + 3 * plane]}, sr, si);
        }
        if (p.finish && sl.w == kCarryWarps - 1) {
            // the last warp's slice ends the scan (empty slices pass the state through)
            p.finish[(size_t)sl.b * 2 * s.C + sl.c] = sr;
            p.finish[(size_t)sl.b * 2 * s.C + s.C + sl.c] = si;
        }
    }
};

// ---------------------------------------------------------------------------
// Forward 3/3: recurrence inside every chunk from its carry; writes read.
//   d_t = v lambda s_{t-1},  s_t = (1 - v) lambda s_{t-1} + gamma v inj
// (field_only_v4_chunked_triton_wiki100.py:599-622).
// ---------------------------------------------------------------------------
template <int VEC, int U>
struct FwdMaterialize {
    using Params = FwdParams;
    static constexpr int kThreads = 32 * kWarpsPerBlock;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const Shape& s = p.s;
        const Tile tl = decode_tile<VEC>(s, block, thread);
        if (!tl.active) return;
        const int C = s.C;
        const Vec<VEC> lr = vec_load<VEC>(p.tr + tl.c0);
        const Vec<VEC> li = vec_load<VEC>(p.ti + tl.c0);
        const Vec<VEC> gm = vec_load<VEC>(p.gamma + tl.c0);
        const size_t plane = (size_t)s.B * s.N * C;
        const size_t cidx = ((size_t)tl.b * s.N + tl.n) * C + tl.c0;
        Vec<VEC> sr = vec_load<VEC>(p.carry + cidx);
        Vec<VEC> si = vec_load<VEC>(p.carry + plane + cidx);

        const float* base = p.raw + (size_t)tl.b * s.L * 3 * C + tl.c0;
        float* obase = p.read + (size_t)tl.b * s.L * 4 * C + tl.c0;
        for (int t0 = tl.tbeg; t0 < tl.tend; t0 += U) {
            Vec<VEC> zr[U], zi[U], zv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 + u < tl.tend) {
                    const float* row = base + (size_t)(t0 + u) * 3 * C;
                    zr[u] = vec_load_stream<VEC>(row);
                    zi[u] = vec_load_stream<VEC>(row + C);
                    zv[u] = vec_load_stream<VEC>(row + 2 * C);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 + u < tl.tend) {
                    Vec<VEC> dr, di;
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const Gate g = make_gate(zr[u].v[k], zi[u].v[k], zv[u].v[k]);
                        float mr, mi;
                        cmul(lr.v[k], li.v[k], sr.v[k], si.v[k], mr, mi);
                        dr.v[k] = g.vac * mr;
                        di.v[k] = g.vac * mi;
                        const float keep = 1.0f - g.vac;
                        const float bs = gm.v[k] * g.vac;
                        sr.v[k] = keep * mr + bs * g.inj_r;
                        si.v[k] = keep * mi + bs * g.inj_i;
                    }
                    float* orow = obase + (size_t)(t0 + u) * 4 * C;
                    vec_store_stream<VEC>(orow, sr);
                    vec_store_stream<VEC>(orow + C, si);
                    vec_store_stream<VEC>(orow + 2 * C, dr);
                    vec_store_stream<VEC>(orow + 3 * C, di);
                }
            }
        }
        if (p.state_out && tl.tend == s.L) {
            float* so = p.state_out + (size_t)tl.b * 2 * C + tl.c0;
            vec_store<VEC>(so, sr);
            vec_store<VEC>(so + C, si);
        }
    }
};

// ---------------------------------------------------------------------------
// Backward 1/3: dual map of every chunk, composed from its last step to its
// first:  carry_{t-1} = conj(a_t) carry_t + q_t,
//         q_t = conj(a_t) u_t + v_t conj(lambda) gd_t
// (field_only_v4_chunked_triton_wiki100.py:655-705). Reads z_v and grad_read.
// ---------------------------------------------------------------------------
template <int VEC, int U>
struct BwdSummary {
    using Params = BwdParams;
    static constexpr int kThreads = 32 * kWarpsPerBlock;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const Shape& s = p.s;
        const Tile tl = decode_tile<VEC>(s, block, thread);
        if (!tl.active) return;
        const int C = s.C;
        const Vec<VEC> lr = vec_load<VEC>(p.tr + tl.c0);
        const Vec<VEC> li = vec_load<VEC>(p.ti + tl.c0);
        Affine m[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) m[k] = affine_identity();

        const float* zbase = p.raw + (size_t)tl.b * s.L * 3 * C + 2 * C + tl.c0;
        const float* gbase = p.grad_read + (size_t)tl.b * s.L * 4 * C + tl.c0;
        for (int t0 = tl.tend; t0 > tl.tbeg; t0 -= U) {
            Vec<VEC> zv[U], ur[U], ui[U], gr[U], gi[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 - 1 - u;
                if (t >= tl.tbeg) {
                    zv[u] = vec_load<VEC>(zbase + (size_t)t * 3 * C);
                    const float* grow = gbase + (size_t)t * 4 * C;
                    ur[u] = vec_load<VEC>(grow);
                    ui[u] = vec_load<VEC>(grow + C);
                    gr[u] = vec_load<VEC>(grow + 2 * C);
                    gi[u] = vec_load<VEC>(grow + 3 * C);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 - 1 - u >= tl.tbeg) {
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const float vac = kVacMax * sigmoidf_fast(zv[u].v[k]);
                        const float keep = 1.0f - vac;
                        // conj(a) as the step's multiplier
                        const float car = keep * lr.v[k];
                        const float cai = -keep * li.v[k];
                        float qr, qi, xr, xi;
                        cmul(car, cai, ur[u].v[k], ui[u].v[k], qr, qi);
                        cmul_conj(lr.v[k], li.v[k], gr[u].v[k], gi[u].v[k], xr, xi);
                        m[k] = affine_then(m[k], car, cai, qr + vac * xr, qi + vac * xi);
                    }
                }
            }
        }
        const size_t plane = (size_t)s.B * s.N * C;
        float* out = p.sum + ((size_t)tl.b * s.N + tl.n) * C + tl.c0;
        Vec<VEC> o0, o1, o2, o3;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            o0.v[k] = m[k].ar; o1.v[k] = m[k].ai; o2.v[k] = m[k].br; o3.v[k] = m[k].bi;
        }
        vec_store<VEC>(out, o0);
        vec_store<VEC>(out + plane, o1);
        vec_store<VEC>(out + 2 * plane, o2);
        vec_store<VEC>(out + 3 * plane, o3);
    }
};

// ---------------------------------------------------------------------------
// Backward 3/3: reverse recurrence inside every chunk; writes grad_raw and the
// chunk's partial parameter gradients
// (field_only_v4_chunked_triton_wiki100.py:794-909):
//   G = u + carry;  da = G conj(s_prev);  m = lambda s_prev
//   dv  = -(lr da_r + li da_i) + gamma (inj . G) + gd . m
//   dlambda += keep da + v gd conj(s_prev);  dgamma += v (inj . G)
//   dz_r = gamma v G_r (1 - inj_r^2);  dz_i likewise;  dz_v = dv 0.9 sig (1 - sig)
//   carry <- conj(a) G + v conj(lambda) gd
// ---------------------------------------------------------------------------
template <int VEC, int U>
struct BwdMaterialize {
    using Params = BwdParams;
    static constexpr int kThreads = 32 * kWarpsPerBlock;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const Shape& s = p.s;
        const Tile tl = decode_tile<VEC>(s, block, thread);
        if (!tl.active) return;
        const int C = s.C;
        const Vec<VEC> lr = vec_load<VEC>(p.tr + tl.c0);
        const Vec<VEC> li = vec_load<VEC>(p.ti + tl.c0);
        const Vec<VEC> gm = vec_load<VEC>(p.gamma + tl.c0);
        const size_t plane = (size_t)s.B * s.N * C;
        const size_t cidx = ((size_t)tl.b * s.N + tl.n) * C + tl.c0;
        Vec<VEC> cr = vec_load<VEC>(p.carry + cidx);
        Vec<VEC> ci = vec_load<VEC>(p.carry + plane + cidx);
        Vec<VEC> dtr = vec_fill<VEC>(0.0f), dti = vec_fill<VEC>(0.0f), dgm = vec_fill<VEC>(0.0f);

        const float* zbase = p.raw + (size_t)tl.b * s.L * 3 * C + tl.c0;
        const float* gbase = p.grad_read + (size_t)tl.b * s.L * 4 * C + tl.c0;
        const float* rbase = p.read + (size_t)tl.b * s.L * 4 * C + tl.c0;
        float* obase = p.grad_raw + (size_t)tl.b * s.L * 3 * C + tl.c0;
        for (int t0 = tl.tend; t0 > tl.tbeg; t0 -= U) {
            Vec<VEC> zr[U], zi[U], zv[U], ur[U], ui[U], gr[U], gi[U], pr[U], pi[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 - 1 - u;
                if (t >= tl.tbeg) {
                    const float* zrow = zbase + (size_t)t * 3 * C;
                    zr[u] = vec_load_stream<VEC>(zrow);
                    zi[u] = vec_load_stream<VEC>(zrow + C);
                    zv[u] = vec_load_stream<VEC>(zrow + 2 * C);
                    const float* grow = gbase + (size_t)t * 4 * C;
                    ur[u] = vec_load_stream<VEC>(grow);
                    ui[u] = vec_load_stream<VEC>(grow + C);
                    gr[u] = vec_load_stream<VEC>(grow + 2 * C);
                    gi[u] = vec_load_stream<VEC>(grow + 3 * C);
                    if (t > 0) {
                        const float* prow = rbase + (size_t)(t - 1) * 4 * C;
                        pr[u] = vec_load_stream<VEC>(prow);
                        pi[u] = vec_load_stream<VEC>(prow + C);
                    } else if (p.state_in) {
                        const float* prow = p.state_in + (size_t)tl.b * 2 * C + tl.c0;
                        pr[u] = vec_load<VEC>(prow);
                        pi[u] = vec_load<VEC>(prow + C);
                    } else {
                        pr[u] = vec_fill<VEC>(0.0f);
                        pi[u] = vec_fill<VEC>(0.0f);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 - 1 - u;
                if (t >= tl.tbeg) {
                    Vec<VEC> ozr, ozi, ozv;
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const Gate g = make_gate(zr[u].v[k], zi[u].v[k], zv[u].v[k]);
                        const float keep = 1.0f - g.vac;
                        const float Gr = ur[u].v[k] + cr.v[k];
                        const float Gi = ui[u].v[k] + ci.v[k];
                        const float gdr = gr[u].v[k], gdi = gi[u].v[k];
                        const float sr = pr[u].v[k], si = pi[u].v[k];
                        float mr, mi, dar, dai, xr, xi, yr, yi, nr, ni;
                        cmul(lr.v[k], li.v[k], sr, si, mr, mi);          // lambda s_prev
                        cmul_conj(sr, si, Gr, Gi, dar, dai);             // G conj(s_prev)
                        cmul_conj(sr, si, gdr, gdi, xr, xi);             // gd conj(s_prev)
                        cmul_conj(lr.v[k], li.v[k], gdr, gdi, yr, yi);   // conj(lambda) gd
                        cmul_conj(keep * lr.v[k], keep * li.v[k], Gr, Gi, nr, ni);  // conj(a) G
                        const float common_b = g.inj_r * Gr + g.inj_i * Gi;
                        const float dv = -lr.v[k] * dar - li.v[k] * dai + gm.v[k] * common_b
                                         + gdr * mr + gdi * mi;
                        dtr.v[k] += keep * dar + g.vac * xr;
                        dti.v[k] += keep * dai + g.vac * xi;
                        dgm.v[k] += g.vac * common_b;
                        const float bs = gm.v[k] * g.vac;
                        ozr.v[k] = bs * Gr * (1.0f - g.inj_r * g.inj_r);
                        ozi.v[k] = bs * Gi * (1.0f - g.inj_i * g.inj_i);
                        ozv.v[k] = dv * kVacMax * g.sig * (1.0f - g.sig);
                        cr.v[k] = nr + g.vac * yr;
                        ci.v[k] = ni + g.vac * yi;
                    }
                    float* orow = obase + (size_t)t * 3 * C;
                    vec_store_stream<VEC>(orow, ozr);
                    vec_store_stream<VEC>(orow + C, ozi);
                    vec_store_stream<VEC>(orow + 2 * C, ozv);
                }
            }
        }
        float* po = p.partial + cidx;
        vec_store<VEC>(po, dtr);
        vec_store<VEC>(po + plane, dti);
        vec_store<VEC>(po + 2 * plane, dgm);
    }
};

// ---------------------------------------------------------------------------
// Backward, last: parameter gradients = sum of the chunk partials over batch and
// chunks, in a fixed order (bitwise reproducible). Block = (plane, 32 channels);
// warp w adds rows w, w + W, ... in double (W = 32), then warp 0 adds the W warp sums.
// Stands for the three tensor.sum(dim=(0,1)) calls of the reference
// (field_only_v4_chunked_triton_wiki100.py:1098-1105).
// ---------------------------------------------------------------------------
constexpr int kReduceWarps = 32;

struct BwdReduce {
    using Params = BwdParams;
    static constexpr int kThreads = 32 * kReduceWarps;
    static constexpr int kPhases = 2;
    static constexpr int kSmemFloats = 2 * kThreads;  // doubles

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int cgroups = (s.C + 31) / 32;
        const int k = block / cgroups;
        const int c = (block % cgroups) * 32 + (thread & 31);
        const int w = thread >> 5;
        double acc = 0.0;
        if (c < s.C) {
            const int rows = s.B * s.N;
            const float* src = p.partial + (size_t)k * rows * s.C + c;
            // rows w, w + W, w + 2W, ...; eight loads in flight, added in row order
            int r = w;
            for (; r + 7 * kReduceWarps < rows; r += 8 * kReduceWarps) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = src[(size_t)(r + j * kReduceWarps) * s.C];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc += (double)v[j];
            }
            for (; r < rows; r += kReduceWarps) acc += (double)src[(size_t)r * s.C];
        }
        reinterpret_cast<double*>(smem)[thread] = acc;
    }

    FL_HD static void phase1(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        if (thread >= 32) return;
        const int cgroups = (s.C + 31) / 32;
        const int k = block / cgroups;
        const int c = (block % cgroups) * 32 + thread;
        if (c >= s.C) return;
        const double* part = reinterpret_cast<const double*>(smem);
        double acc = 0.0;
        for (int w = 0; w < kReduceWarps; ++w) acc += part[w * 32 + thread];
        float* dst = k == 0 ? p.grad_tr : (k == 1 ? p.grad_ti : p.grad_gamma);
        dst[c] = (float)acc;
    }
};

// ---------------------------------------------------------------------------
// Span summary: the affine map of a whole span per (batch, channel), composed from
// the chunk maps that FwdSummary wrote. One block owns 32 channels of one batch row;
// warp w composes its slice of chunks (phase 0), warp 0 composes the slices (phase 1).
// This pair is what sequence-sharded ranks exchange.
// ---------------------------------------------------------------------------
struct SpanCompose {
    struct Params {
        const float* sum;  // [4][B][N][C]
        float* summary;    // [B][4][C]  Re A | Im A | Re B | Im B
        Shape s;
        int reverse;       // non-zero: compose from the last chunk to the first (dual maps)
    };
    static constexpr int kThreads = 32 * kCarryWarps;
    static constexpr int kPhases = 2;
    static constexpr int kSmemFloats = 4 * kThreads;

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int cgroups = (s.C + 31) / 32;
        const int lane = thread & 31, w = thread >> 5;
        const int b = block / cgroups;
        const int c = (block % cgroups) * 32 + lane;
        if (c >= s.C) return;
        const int per = (s.N + kCarryWarps - 1) / kCarryWarps;
        const int lo = w * per < s.N ? w * per : s.N;
        const int hi = lo + per < s.N ? lo + per : s.N;
        const size_t plane = (size_t)s.B * s.N * s.C;
        // position i in composition order is chunk i, or chunk N-1-i when composing backwards
        const int first = p.reverse ? s.N - 1 : 0, step = p.reverse ? -1 : 1;
        Affine m = affine_identity();
        int i = lo;
        for (; i + 8 <= hi; i += 8) {  // eight maps in flight, composed in order
            float v[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const size_t idx = ((size_t)b * s.N + first + step * (i + j)) * s.C + c;
                v[j][0] = p.sum[idx]; v[j][1] = p.sum[idx + plane];
                v[j][2] = p.sum[idx + 2 * plane]; v[j][3] = p.sum[idx + 3 * plane];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) m = affine_then(m, v[j][0], v[j][1], v[j][2], v[j][3]);
        }
        for (; i < hi; ++i) {
            const size_t idx = ((size_t)b * s.N + first + step * i) * s.C + c;
            m = affine_then(m, p.sum[idx], p.sum[idx + plane], p.sum[idx + 2 * plane],
                            p.sum[idx + 3 * plane]);
        }
        float* o = smem + 4 * thread;
        o[0] = m.ar; o[1] = m.ai; o[2] = m.br; o[3] = m.bi;
    }

    FL_HD static void phase1(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        if (thread >= 32) return;
        const int cgroups = (s.C + 31) / 32;
        const int b = block / cgroups;
        const int c = (block % cgroups) * 32 + thread;
        if (c >= s.C) return;
        Affine m = affine_identity();
        for (int w = 0; w < kCarryWarps; ++w) {
            const float* q = smem + 4 * (w * 32 + thread);
            m = affine_then(m, q[0], q[1], q[2], q[3]);
        }
        float* o = p.summary + (size_t)b * 4 * s.C + c;
        o[0] = m.ar; o[s.C] = m.ai; o[2 * s.C] = m.br; o[3 * s.C] = m.bi;
    }
};

// ---------------------------------------------------------------------------
// Fold of the span summaries of the ranks before `rank` onto the sequence's initial
// state: the state entering rank's span. One thread per (batch, channel).
// ---------------------------------------------------------------------------
struct FoldSummaries {
    struct Params {
        const float* summaries;  // [P][B][4][C]
        const float* state0;     // [B, 2C] or null: state before the first span
        float* state;            // [B, 2C]
        int rank, P, B, C;
        int reverse;  // non-zero: fold the ranks AFTER `rank`, last first (gradient carry)
    };
    static constexpr int kThreads = 128;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const long long i = (long long)block * kThreads + thread;
        if (i >= (long long)p.B * p.C) return;
        const int b = (int)(i / p.C), c = (int)(i % p.C);
        float sr = p.state0 ? p.state0[(size_t)b * 2 * p.C + c] : 0.0f;
        float si = p.state0 ? p.state0[(size_t)b * 2 * p.C + p.C + c] : 0.0f;
        const int count = p.reverse ? p.P - 1 - p.rank : p.rank;
        for (int k = 0; k < count; ++k) {
            const int r = p.reverse ? p.P - 1 - k : k;
            const float* m = p.summaries + (((size_t)r * p.B + b) * 4) * p.C + c;
            affine_apply(Affine{m[0], m[p.C], m[2 * (size_t)p.C], m[3 * (size_t)p.C]}, sr, si);
        }
        p.state[(size_t)b * 2 * p.C + c] = sr;
        p.state[(size_t)b * 2 * p.C + p.C + c] = si;
    }
};


// ---------------------------------------------------------------------------
// One recurrent step for incremental decoding: the state is carried by the caller,
// one token per sequence enters, one row of `read` comes out. One thread per
// (sequence, channel); all accesses coalesced over channels. The arithmetic is one
// iteration of the forward recurrence (reference :599-622); the reference itself has no
// incremental path, its full-sequence forward over prefix + new tokens is the oracle.
// IO = float or bf16 bits (uint16_t) for raw and read; the state is always fp32.
// ---------------------------------------------------------------------------
FL_HD float io_load(const float* p, size_t i) { return p[i]; }
FL_HD float io_load(const uint16_t* p, size_t i) { return bf16_bits_to_float(p[i]); }
FL_HD void io_store(float* p, size_t i, float v) { p[i] = v; }
FL_HD void io_store(uint16_t* p, size_t i, float v) { p[i] = float_to_bf16_bits(v); }

template <typename IO>
struct DecodeStep {
    struct Params {
        const IO* raw;  // [B, 3C]
        const float* tr;
        const float* ti;
        const float* gamma;
        float* state;   // [B, 2C] in and out
        IO* read;       // [B, 4C]
        int B, C;
    };
    static constexpr int kThreads = 128;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const long long i = (long long)block * kThreads + thread;
        if (i >= (long long)p.B * p.C) return;
        const int b = (int)(i / p.C), c = (int)(i % p.C);
        const size_t C = p.C;
        const Gate g = make_gate(io_load(p.raw, b * 3 * C + c), io_load(p.raw, b * 3 * C + C + c),
                                 io_load(p.raw, b * 3 * C + 2 * C + c));
        float sr = p.state[b * 2 * C + c], si = p.state[b * 2 * C + C + c];
        float mr, mi;
        cmul(p.tr[c], p.ti[c], sr, si, mr, mi);
        const float bs = p.gamma[c] * g.vac;
        sr = (1.0f - g.vac) * mr + bs * g.inj_r;
        si = (1.0f - g.vac) * mi + bs * g.inj_i;
        p.state[b * 2 * C + c] = sr;
        p.state[b * 2 * C + C + c] = si;
        io_store(p.read, b * 4 * C + c, sr);
        io_store(p.read, b * 4 * C + C + c, si);
        io_store(p.read, b * 4 * C + 2 * C + c, g.vac * mr);
        io_store(p.read, b * 4 * C + 3 * C + c, g.vac * mi);
    }
};

}  // namespace fields
