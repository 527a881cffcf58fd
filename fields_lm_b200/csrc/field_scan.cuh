// Real-valued first-order scan  s_t = a_t s_{t-1} + x_t  over [B, L, C], forward and backward.
//
// The second call site of the reference's scan primitive: `hierarchical_scan(a, drive, block=32)`
// (field_only_v4_chunked_triton_wiki100.py:347-391) as the softpatch mixer calls it on a rank-64
// state (official_source/field_hybrid_speed_optimization_v6.py:333-335), where `a` is one decay per
// token broadcast over the channels. The reference computes it with a log-depth doubling scan
// inside blocks of 32 and a second doubling scan over the blocks; here it is the same three steps
// as chunk maps -> carries -> states, each step walked sequentially by the thread that owns a
// (chunk, channel), which is also what the fp32 oracle does.
//
// Work layout: a warp owns one chunk of kScanChunk steps of 32 channels (a lane per channel, so a
// row of a plane is one 128-byte line per warp); blocks hold kScanWarps such items. The tensors of
// this call site are a few MB, all of it L2-resident after the first touch; the kernels are sized
// for launch latency, not for HBM.
//
// Backward (g = grad of the states, c = carry from the later steps, c_{L-1} = grad_state_out):
//   lambda_t = g_t + c_t,  grad_x_t = lambda_t,  grad_a_t = lambda_t s_{t-1},  c_{t-1} = a_t lambda_t.
#pragma once

#include "field_math.cuh"

namespace fields {

constexpr int kScanChunk = 16;   // steps per chunk
constexpr int kScanWarps = 4;    // chunks of 32 channels per block
constexpr int kScanUnroll = 8;   // loads issued together while walking a chunk

// `a` may be a broadcast view: element (b, t, c) is a[b * a_batch + t * a_step + c * a_chan].
struct ScanShape {
    int B, L, C;
    int NT;   // chunks per sequence
    int CG;   // groups of 32 channels
    long long a_batch, a_step;
    int a_chan;
};

struct ScanItem {
    int b, n, c;   // batch row, chunk, channel of this lane
    int t0, t1;    // the chunk's steps [t0, t1)
    bool ok;
};

FL_HD ScanItem scan_item(const ScanShape& s, int block, int thread) {
    const long long item = (long long)block * kScanWarps + (thread >> 5);
    ScanItem it;
    const int cg = (int)(item % s.CG);
    const long long rest = item / s.CG;
    it.n = (int)(rest % s.NT);
    it.b = (int)(rest / s.NT);
    it.c = cg * 32 + (thread & 31);
    it.t0 = it.n * kScanChunk;
    it.t1 = it.t0 + kScanChunk < s.L ? it.t0 + kScanChunk : s.L;
    it.ok = it.b < s.B && it.c < s.C;
    return it;
}

FL_HD long long scan_items(const ScanShape& s) { return (long long)s.B * s.NT * s.CG; }

struct ScanFwdParams {
    const float* a;
    const float* x;          // drive [B, L, C]
    const float* state_in;   // [B, C] or null (zero)
    float* states;           // [B, L, C]
    float* state_out;        // [B, C] or null
    float* map_a;            // [B, NT, C]
    float* map_b;            // [B, NT, C]
    float* carry;            // [B, NT, C] state entering each chunk
    ScanShape s;
};

// Chunk maps: s_end = A s_begin + B over the chunk's steps (reference :364-377, sequentially).
struct ScanChunkMap {
    using Params = ScanFwdParams;
    static constexpr int kThreads = 32 * kScanWarps;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const ScanItem it = scan_item(s, block, thread);
        if (!it.ok) return;
        const float* ap = p.a + it.b * s.a_batch + (long long)it.c * s.a_chan;
        const float* xp = p.x + (size_t)it.b * s.L * s.C + it.c;
        float A = 1.0f, Bv = 0.0f;
        for (int t = it.t0; t < it.t1; t += kScanUnroll) {
            float av[kScanUnroll], xv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t + u < it.t1) {
                    av[u] = ap[(t + u) * s.a_step];
                    xv[u] = xp[(size_t)(t + u) * s.C];
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t + u < it.t1) {
                    A *= av[u];
                    Bv = av[u] * Bv + xv[u];
                }
            }
        }
        const size_t o = ((size_t)it.b * s.NT + it.n) * s.C + it.c;
        p.map_a[o] = A;
        p.map_b[o] = Bv;
    }
};

// Carries: the state entering every chunk (reference :382-386), one thread per (row, channel).
struct ScanCarry {
    using Params = ScanFwdParams;
    static constexpr int kThreads = 128;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const long long i = (long long)block * kThreads + thread;
        if (i >= (long long)s.B * s.C) return;
        const int b = (int)(i / s.C), c = (int)(i % s.C);
        float st = p.state_in ? p.state_in[(size_t)b * s.C + c] : 0.0f;
        const size_t base = (size_t)b * s.NT * s.C + c;
        for (int n = 0; n < s.NT; n += kScanUnroll) {
            float A[kScanUnroll], Bv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (n + u < s.NT) {
                    A[u] = p.map_a[base + (size_t)(n + u) * s.C];
                    Bv[u] = p.map_b[base + (size_t)(n + u) * s.C];
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (n + u < s.NT) {
                    p.carry[base + (size_t)(n + u) * s.C] = st;
                    st = A[u] * st + Bv[u];
                }
            }
        }
    }
};

// States: every chunk again from its entering state (reference :387).
struct ScanEmit {
    using Params = ScanFwdParams;
    static constexpr int kThreads = 32 * kScanWarps;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const ScanItem it = scan_item(s, block, thread);
        if (!it.ok) return;
        const float* ap = p.a + it.b * s.a_batch + (long long)it.c * s.a_chan;
        const float* xp = p.x + (size_t)it.b * s.L * s.C + it.c;
        float* op = p.states + (size_t)it.b * s.L * s.C + it.c;
        float st = p.carry[((size_t)it.b * s.NT + it.n) * s.C + it.c];
        for (int t = it.t0; t < it.t1; t += kScanUnroll) {
            float av[kScanUnroll], xv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t + u < it.t1) {
                    av[u] = ap[(t + u) * s.a_step];
                    xv[u] = xp[(size_t)(t + u) * s.C];
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t + u < it.t1) {
                    st = av[u] * st + xv[u];
                    op[(size_t)(t + u) * s.C] = st;
                }
            }
        }
        // the outgoing state is the last emitted state, bit for bit
        if (p.state_out && it.n == s.NT - 1) p.state_out[(size_t)it.b * s.C + it.c] = st;
    }
};

struct ScanBwdParams {
    const float* a;
    const float* states;          // forward output [B, L, C]
    const float* state_in;        // [B, C] or null
    const float* grad_states;     // [B, L, C]
    const float* grad_state_out;  // [B, C] or null
    float* grad_a;                // [B, L, C] (dense, also for a broadcast `a`)
    float* grad_x;                // [B, L, C]
    float* grad_state_in;         // [B, C] or null
    float* map_a;
    float* map_b;
    float* carry;                 // carry entering each chunk from the later steps
    ScanShape s;
};

// Dual chunk maps: c_before = A c_after + B, walking the chunk from its last step to its first.
struct ScanChunkMapBwd {
    using Params = ScanBwdParams;
    static constexpr int kThreads = 32 * kScanWarps;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const ScanItem it = scan_item(s, block, thread);
        if (!it.ok) return;
        const float* ap = p.a + it.b * s.a_batch + (long long)it.c * s.a_chan;
        const float* gp = p.grad_states + (size_t)it.b * s.L * s.C + it.c;
        float A = 1.0f, Bv = 0.0f;
        for (int t = it.t1 - 1; t >= it.t0; t -= kScanUnroll) {
            float av[kScanUnroll], gv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t - u >= it.t0) {
                    av[u] = ap[(t - u) * s.a_step];
                    gv[u] = gp[(size_t)(t - u) * s.C];
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (t - u >= it.t0) {
                    A *= av[u];
                    Bv = av[u] * (Bv + gv[u]);
                }
            }
        }
        const size_t o = ((size_t)it.b * s.NT + it.n) * s.C + it.c;
        p.map_a[o] = A;
        p.map_b[o] = Bv;
    }
};

struct ScanCarryBwd {
    using Params = ScanBwdParams;
    static constexpr int kThreads = 128;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const long long i = (long long)block * kThreads + thread;
        if (i >= (long long)s.B * s.C) return;
        const int b = (int)(i / s.C), c = (int)(i % s.C);
        float cr = p.grad_state_out ? p.grad_state_out[(size_t)b * s.C + c] : 0.0f;
        const size_t base = (size_t)b * s.NT * s.C + c;
        for (int n = s.NT - 1; n >= 0; n -= kScanUnroll) {
            float A[kScanUnroll], Bv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (n - u >= 0) {
                    A[u] = p.map_a[base + (size_t)(n - u) * s.C];
                    Bv[u] = p.map_b[base + (size_t)(n - u) * s.C];
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                if (n - u >= 0) {
                    p.carry[base + (size_t)(n - u) * s.C] = cr;
                    cr = A[u] * cr + Bv[u];
                }
            }
        }
    }
};

struct ScanEmitBwd {
    using Params = ScanBwdParams;
    static constexpr int kThreads = 32 * kScanWarps;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;
    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const ScanShape& s = p.s;
        const ScanItem it = scan_item(s, block, thread);
        if (!it.ok) return;
        const float* ap = p.a + it.b * s.a_batch + (long long)it.c * s.a_chan;
        const size_t row0 = (size_t)it.b * s.L * s.C + it.c;
        const float* gp = p.grad_states + row0;
        const float* sp = p.states + row0;
        float* gxp = p.grad_x + row0;
        float* gap = p.grad_a + row0;
        const float first = p.state_in ? p.state_in[(size_t)it.b * s.C + it.c] : 0.0f;
        float cr = p.carry[((size_t)it.b * s.NT + it.n) * s.C + it.c];
        for (int t = it.t1 - 1; t >= it.t0; t -= kScanUnroll) {
            float av[kScanUnroll], gv[kScanUnroll], pv[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                const int tt = t - u;
                if (tt >= it.t0) {
                    av[u] = ap[tt * s.a_step];
                    gv[u] = gp[(size_t)tt * s.C];
                    pv[u] = tt > 0 ? sp[(size_t)(tt - 1) * s.C] : first;
                }
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                const int tt = t - u;
                if (tt >= it.t0) {
                    const float lam = gv[u] + cr;
                    gxp[(size_t)tt * s.C] = lam;
                    gap[(size_t)tt * s.C] = lam * pv[u];
                    cr = av[u] * lam;
                }
            }
        }
        if (p.grad_state_in && it.n == 0) p.grad_state_in[(size_t)it.b * s.C + it.c] = cr;
    }
};

}  // namespace fields
