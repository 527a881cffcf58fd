// Single-pass Field kernels: every input is read from HBM once and every output
// written once; the carry between time tiles is resolved inside the kernel by a
// decoupled look-back over per-tile aggregates published in global memory
// (field_sync.cuh).
//
// A block owns one tile = (batch row, 128-channel group, TT = WARPS * TS time steps).
// Warp w owns TS consecutive steps of the tile, a lane owns 4 consecutive channels
// (128-bit accesses, 512 contiguous bytes per warp per plane and step). Tiles are taken
// in block-index order, time-major, so every tile a block may wait for belongs to a
// block with a smaller index, which the hardware has already started.
//
// Forward, per block:
//   1. load the warp's TS steps into registers, turn them into (b_r, b_i, vacancy) in
//      place and compose the warp's affine map (gates: reference :493-501);
//   2. 128 threads (one per channel) compose the tile's map from the warp maps and
//      publish it, then walk back over earlier tiles of the chain, composing published
//      aggregates until they meet a tile whose end state is known, which gives the state
//      entering this tile; they publish this tile's end state;
//   3. every warp runs the recurrence over its registers from its incoming state and
//      writes read = [Re s | Im s | Re d | Im d] (reference :599-622).
// Every wait is bounded; on expiry the block records an error word, poisons its carry
// with NaN and carries on, so the kernel always terminates.
//
// Kernel bodies are split into phases. Per-thread values that live across phases sit in
// a State struct: registers on the device, an array per block in the host emulation
// used by the CPU tests.
#pragma once

#include "field_kernels.cuh"
#include "field_sync.cuh"

namespace fields {

constexpr int kCtrlHeader = 64;  // unsigned words before the slots: [0] error word
constexpr int kGroup = 128;      // channels per tile

struct SpShape {
    int B, L, C;
    int NT;        // time tiles per chain
    int G;         // 128-channel groups
    int prefetch;  // non-zero: blocks warm L2 with the inputs of the tile that many positions ahead
    unsigned max_polls;  // bound of every wait for another block's publication
    int ticket;    // non-zero: blocks take their tile from a counter in the workspace header
};

// Prefetches `planes` consecutive 128-channel plane chunks of `steps` rows into L2:
// row r, plane q is the 128 elements at base + r * row_floats + q * plane_floats.
template <typename T>
FL_HD void prefetch_rows(const T* base, int steps, int valid_steps, int planes, size_t row_floats,
                         size_t plane_floats, int valid_floats, int thread, int threads) {
    constexpr int kPerLine = 128 / (int)sizeof(T);   // elements per 128-byte line
    constexpr int kLines = 128 / kPerLine;           // lines per 128-channel chunk
    const int lines = steps * planes * kLines;
    for (int q = thread; q < lines; q += threads) {
        const int t = q / (planes * kLines);
        const int r = q % (planes * kLines);
        const int plane = r / kLines, line = r % kLines;
        if (t < valid_steps && line * kPerLine < valid_floats)
            prefetch_l2(base + (size_t)t * row_floats + (size_t)plane * plane_floats + line * kPerLine);
    }
}

template <typename IO>
struct SpFwdParamsT {
    const IO* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;  // [B, 2C] or null
    IO* read;
    float* state_out;       // [B, 2C] or null
    float* agg;             // [tiles][128][4]  tile maps (Re A, Im A, Re B, Im B)
    float* incl;            // [tiles][128][2]  state after each tile
    unsigned* ctrl;         // error word; filled with 0xFF like the slots before the launch
    SpShape s;
    // Kernels built with STATS also write, per token and 128-channel group, the sum of squares of
    // the four output planes (fp32 values, before any rounding of `read`): [B, L, G].
    float* sumsq = nullptr;
};
using SpFwdParams = SpFwdParamsT<float>;

struct SpTile {
    int b, cg, n;        // batch row, channel group, position in scan order
    long long chain;     // b * G + cg
    long long idx;       // chain * NT + n : slot index into agg / incl
};

FL_HD SpTile sp_decode(const SpShape& s, unsigned ticket) {
    SpTile t;
    const long long chains = (long long)s.B * s.G;
    t.n = (int)(ticket / chains);
    t.chain = ticket % chains;
    t.b = (int)(t.chain / s.G);
    t.cg = (int)(t.chain % s.G);
    t.idx = t.chain * s.NT + t.n;
    return t;
}

// IO = float, or uint16_t for bfloat16 raw / read (the state, the maps and all arithmetic stay fp32).
//
// STAGED: the kernel runs as persistent blocks that take their tiles from a ticket counter in the
// workspace header, one tile ahead: while a block works on a tile it already holds the ticket
// of its next one. Every thread keeps one staging cell per (step, plane) of its rows in shared
// memory; once the block has moved the current tile's rows from the cells into registers
// (phase 0) every thread starts the cp.async copies of its rows of the NEXT tile into the same
// cells. They land while the block publishes its map, looks back and runs the recurrence, so the
// next tile starts from shared memory instead of waiting for HBM. Tickets are taken in time-major
// tile order by blocks that are running, so every tile a block waits for is held by a running
// block (as its current or its next tile): progress does not depend on how many blocks the GPU
// holds at once or on the order it starts them in. The atomic of a ticket is issued at the top
// of a tile and its result is used after phase 0, so its latency is off the critical path.
// (Holding two tickets ahead, so that a thread could start the next tile's copies right after
// its own cell loads, was measured and was much slower: 80 us against 43 us. A ticket taken
// early is a tile that its chain's successors wait for while its block is still busy.)
template <int TS, int WARPS, int MIN_BLOCKS, typename IO = float, bool STATS = false,
          bool STAGED = false>
struct FwdSinglePass {
    using Params = SpFwdParamsT<IO>;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;  // blocks per SM that the register count must allow
    static constexpr int kTile = TS * WARPS;
    static constexpr int kPhases = STATS ? 5 : 4;
    static constexpr int kStatRow = 33;  // lane partials of one (warp, step), padded against bank conflicts
    static_assert(!STATS || kTile * kStatRow <= WARPS * 4 * kGroup, "lane partials reuse the map area");
    static constexpr int kSplitPhase = 2;  // host emulation: phases < 2 of all blocks run first
    static constexpr int kSumFloats = WARPS * 4 * kGroup;
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;
    static constexpr bool kStaged = STAGED;
    static constexpr int kCellFloats = (int)sizeof(IO);  // four elements: 16 bytes of float, 8 of bfloat16
    static constexpr int kStageFloats = STAGED ? TS * 3 * kThreads * kCellFloats : 0;
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kStageFloats + (STAGED ? 4 : 0);
    // the word through which thread 0 hands the block's next ticket to the other threads
    FL_HD static unsigned* ticket_at(float* smem) {
        return reinterpret_cast<unsigned*>(smem + kSumFloats + kCarryFloats + kStageFloats);
    }
    static constexpr int kClaimAfter = 2;  // the next tile is claimed after the look-back phase
    FL_HD static constexpr bool barrier_after(int ph) { return ph != 1; }
    FL_HD static float* cell_at(float* smem, int idx, int thread) {
        return smem + kSumFloats + kCarryFloats + ((size_t)idx * kThreads + thread) * kCellFloats;
    }

    // Starts the copies of this thread's rows of `tile` into its staging cells (one commit group).
    FL_HD static void stage(const Params& p, int tile, int thread, float* smem) {
        const SpShape& s = p.s;
        const SpTile tl = sp_decode(s, (unsigned)tile);
        const int lane = thread & 31, warp = thread >> 5;
        const int c0 = tl.cg * kGroup + lane * 4;
        if (c0 < s.C) {
            const int tw = tl.n * kTile + warp * TS;
            const IO* base = p.raw + ((size_t)tl.b * s.L) * 3 * s.C + c0;
#pragma unroll
            for (int u = 0; u < TS; ++u) {
                if (tw + u < s.L) {
                    const IO* row = base + (size_t)(tw + u) * 3 * s.C;
                    async_copy4(cell_at(smem, u * 3 + 0, thread), row);
                    async_copy4(cell_at(smem, u * 3 + 1, thread), row + s.C);
                    async_copy4(cell_at(smem, u * 3 + 2, thread), row + 2 * s.C);
                }
            }
        }
        async_commit();
    }

    struct State {
        Vec<4> br[TS], bi[TS], vac[TS];  // raw on load, then gamma*v*inj and vacancy
    };

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }

    // Warms L2 with the raw rows of the tile this block will process next.
    FL_HD static void prefetch(const Params& p, int tile, int thread) {
        const SpShape& s = p.s;
        const SpTile nx = sp_decode(s, (unsigned)tile);
        const int t0 = nx.n * kTile;
        prefetch_rows(p.raw + ((size_t)nx.b * s.L + t0) * 3 * s.C + nx.cg * kGroup, kTile, s.L - t0, 3,
                      (size_t)3 * s.C, (size_t)s.C, s.C - nx.cg * kGroup, thread, kThreads);
    }

    template <int PH>
    FL_HD static void phase(const Params& p, int block, int thread, float* smem, State& st) {
        const SpShape& s = p.s;
        const SpTile tl = sp_decode(s, (unsigned)block);
        const int lane = thread & 31, warp = thread >> 5;
        const int C = s.C;
        const int c0 = tl.cg * kGroup + lane * 4;
        const bool chan_ok = c0 < C;
        const int tw = tl.n * kTile + warp * TS;

        if constexpr (PH == 0) {
            Affine m[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) m[k] = affine_identity();
            if constexpr (STAGED) {
                // The rows were started into this thread's cells by the kernel entry while the
                // block's previous tile ran (by this very call in the host emulation, where a
                // copy is synchronous).
#if !FL_DEVICE_CODE
                stage(p, block, thread, smem);
#endif
                async_wait_pending<0>();
                if (chan_ok) {
#pragma unroll
                    for (int u = 0; u < TS; ++u) {
                        if (tw + u < s.L) {
                            st.br[u] = cell_load4<IO>(cell_at(smem, u * 3 + 0, thread));
                            st.bi[u] = cell_load4<IO>(cell_at(smem, u * 3 + 1, thread));
                            st.vac[u] = cell_load4<IO>(cell_at(smem, u * 3 + 2, thread));
                        }
                    }
                }
                // (on the device the kernel entry starts the next tile's rows towards the cells
                // after the barrier that follows this phase)
            }
            if (chan_ok) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                if constexpr (!STAGED) {
                    const IO* base = p.raw + ((size_t)tl.b * s.L) * 3 * C + c0;
#pragma unroll
                    for (int u = 0; u < TS; ++u) {
                        if (tw + u < s.L) {
                            const IO* row = base + (size_t)(tw + u) * 3 * C;
                            st.br[u] = io_load4_stream(row);
                            st.bi[u] = io_load4_stream(row + C);
                            st.vac[u] = io_load4_stream(row + 2 * C);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < TS; ++u) {
                    if (tw + u < s.L) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const Gate g = make_gate(st.br[u].v[k], st.bi[u].v[k], st.vac[u].v[k]);
                            const float keep = 1.0f - g.vac;
                            const float bs = gm.v[k] * g.vac;
                            st.br[u].v[k] = bs * g.inj_r;
                            st.bi[u].v[k] = bs * g.inj_i;
                            st.vac[u].v[k] = g.vac;
                            m[k] = affine_then(m[k], keep * lr.v[k], keep * li.v[k],
                                               st.br[u].v[k], st.bi[u].v[k]);
                        }
                    }
                }
            }
            Vec<4> o0, o1, o2, o3;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o0.v[k] = m[k].ar; o1.v[k] = m[k].ai; o2.v[k] = m[k].br; o3.v[k] = m[k].bi;
            }
            vec_store<4>(sum_at(smem, warp, 0) + lane * 4, o0);
            vec_store<4>(sum_at(smem, warp, 1) + lane * 4, o1);
            vec_store<4>(sum_at(smem, warp, 2) + lane * 4, o2);
            vec_store<4>(sum_at(smem, warp, 3) + lane * 4, o3);
        } else if constexpr (PH == 1) {
            // tile aggregate, one thread per channel; the first tile of a chain publishes
            // only its end state
            if (thread < kGroup && tl.cg * kGroup + thread < C && tl.n > 0) {
                Affine a = affine_identity();
#pragma unroll
                for (int w = 0; w < WARPS; ++w)
                    a = affine_then(a, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                    sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
                publish4(p.agg + ((size_t)tl.idx * kGroup + thread) * 4, a.ar, a.ai, a.br, a.bi);
            }
        } else if constexpr (PH == 2) {
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                float sr, si;
                if (tl.n == 0) {
                    sr = p.state_in ? p.state_in[(size_t)tl.b * 2 * C + ch] : 0.0f;
                    si = p.state_in ? p.state_in[(size_t)tl.b * 2 * C + C + ch] : 0.0f;
                } else {
                    look_back(p.agg, p.incl, tl.chain * s.NT, tl.n, thread, p.ctrl, s.max_polls, sr, si);
                }
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    carry_at(smem, w, 0)[thread] = sr;
                    carry_at(smem, w, 1)[thread] = si;
                    affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                        sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                                 sr, si);
                }
                publish2(p.incl + ((size_t)tl.idx * kGroup + thread) * 2, sr, si);
                if (p.state_out && tl.n == s.NT - 1) {
                    p.state_out[(size_t)tl.b * 2 * C + ch] = sr;
                    p.state_out[(size_t)tl.b * 2 * C + C + ch] = si;
                }
            }
        } else if constexpr (PH == 3) {
            if (!chan_ok) {
                if constexpr (STATS) {
#pragma unroll
                    for (int u = 0; u < TS; ++u) smem[(warp * TS + u) * kStatRow + lane] = 0.0f;
                }
                return;
            }
            const Vec<4> lr = vec_load<4>(p.tr + c0);
            const Vec<4> li = vec_load<4>(p.ti + c0);
            Vec<4> sr = vec_load<4>(carry_at(smem, warp, 0) + lane * 4);
            Vec<4> si = vec_load<4>(carry_at(smem, warp, 1) + lane * 4);
            IO* obase = p.read + ((size_t)tl.b * s.L) * 4 * C + c0;
#pragma unroll
            for (int u = 0; u < TS; ++u) {
                if (tw + u < s.L) {
                    Vec<4> dr, di;
                    float sq = 0.0f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float mr, mi;
                        cmul(lr.v[k], li.v[k], sr.v[k], si.v[k], mr, mi);
                        const float v = st.vac[u].v[k];
                        dr.v[k] = v * mr;
                        di.v[k] = v * mi;
                        sr.v[k] = (1.0f - v) * mr + st.br[u].v[k];
                        si.v[k] = (1.0f - v) * mi + st.bi[u].v[k];
                        if constexpr (STATS)
                            sq += sr.v[k] * sr.v[k] + si.v[k] * si.v[k] + dr.v[k] * dr.v[k] +
                                  di.v[k] * di.v[k];
                    }
                    IO* orow = obase + (size_t)(tw + u) * 4 * C;
                    io_store4_stream(orow, sr);
                    io_store4_stream(orow + C, si);
                    io_store4_stream(orow + 2 * C, dr);
                    io_store4_stream(orow + 3 * C, di);
                    // the map area is free after the look-back: one partial per lane and step
                    if constexpr (STATS) smem[(warp * TS + u) * kStatRow + lane] = sq;
                }
            }
        } else {  // PH == 4 (STATS): one sum per step of the tile, lanes added in order
            if (thread < kTile) {
                const int t = tl.n * kTile + thread;  // thread = warp * TS + step
                if (t < s.L) {
                    float acc = 0.0f;
#pragma unroll
                    for (int l = 0; l < 32; ++l) acc += smem[thread * kStatRow + l];
                    p.sumsq[((size_t)tl.b * s.L + t) * s.G + tl.cg] = acc;
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------
// Forward in two sweeps per tile with asynchronous rings (the shape of the backward
// below): sweep 1 streams the tile's raw rows through per-thread cp.async rings, evaluates
// the gates and composes the warp's map; after the look-back, sweep 2 streams the same rows
// again (now from L2), evaluates the gates a second time and runs the recurrence, writing
// read. Nothing of the tile lives in registers between the sweeps, so more warps fit on an
// SM and loads are always in flight; the price is the second gate evaluation. HBM traffic
// stays compulsory: the second read is served by L2.
// ---------------------------------------------------------------------------
template <int TS, int WARPS, int U_, int MIN_BLOCKS, int STAGES, typename IO = float>
struct FwdTwoSweep {
    using Params = SpFwdParamsT<IO>;
    static constexpr bool kStaged = false;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kPhases = 4;
    static constexpr int kSplitPhase = 2;
    static constexpr int kClaimAfter = 2;
    static constexpr int U = U_;
    static constexpr int kSumFloats = WARPS * 4 * kGroup;
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;
    static constexpr int kCells = U * 3;
    static constexpr int kRingFloats = STAGES * kCells * kThreads * 4;
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kRingFloats;
    static_assert(kThreads >= kGroup, "one thread per channel is needed for the look-back");
    FL_HD static constexpr bool barrier_after(int ph) { return ph != 1; }

    struct State {};

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }
    FL_HD static float* cell_at(float* smem, int stage, int idx, int thread) {
        return smem + kSumFloats + kCarryFloats +
               ((size_t)(stage * kCells + idx) * kThreads + thread) * 4;
    }

    FL_HD static void prefetch(const Params&, int, int) {}

    template <int PH>
    FL_HD static void phase(const Params& p, int block, int thread, float* smem, State&) {
        const SpShape& s = p.s;
        const SpTile tl = sp_decode(s, (unsigned)block);
        const int lane = thread & 31, warp = thread >> 5;
        const int C = s.C;
        const int c0 = tl.cg * kGroup + lane * 4;
        const bool chan_ok = c0 < C;
        const int tfirst = tl.n * kTile + warp * TS;
        const int tbeg = tfirst < s.L ? tfirst : s.L;
        const int tend = tbeg + TS < s.L ? tbeg + TS : s.L;
        const IO* base = p.raw + ((size_t)tl.b * s.L) * 3 * C + c0;

        // batch of U steps starting at t0 into ring slot `stage` (nothing past tend)
        auto issue = [&](int t0, int stage) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 + u;
                if (t < tend) {
                    const IO* row = base + (size_t)t * 3 * C;
                    async_copy4(cell_at(smem, stage, u * 3 + 0, thread), row);
                    async_copy4(cell_at(smem, stage, u * 3 + 1, thread), row + C);
                    async_copy4(cell_at(smem, stage, u * 3 + 2, thread), row + 2 * C);
                }
            }
            async_commit();
        };

        if constexpr (PH == 0) {
            Affine m[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) m[k] = affine_identity();
            if (chan_ok) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
#pragma unroll
                for (int j = 0; j < STAGES - 1; ++j) issue(tbeg + j * U, j);
                int stage = 0;
                for (int t0 = tbeg; t0 < tend; t0 += U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                    issue(t0 + (STAGES - 1) * U, stage == 0 ? STAGES - 1 : stage - 1);
                    async_wait_pending<STAGES - 1>();
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (t0 + u < tend) {
                            const Vec<4> zr = cell_load4<IO>(cell_at(smem, stage, u * 3 + 0, thread));
                            const Vec<4> zi = cell_load4<IO>(cell_at(smem, stage, u * 3 + 1, thread));
                            const Vec<4> zv = cell_load4<IO>(cell_at(smem, stage, u * 3 + 2, thread));
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const Gate g = make_gate(zr.v[k], zi.v[k], zv.v[k]);
                                const float keep = 1.0f - g.vac;
                                const float bs = gm.v[k] * g.vac;
                                m[k] = affine_then(m[k], keep * lr.v[k], keep * li.v[k],
                                                   bs * g.inj_r, bs * g.inj_i);
                            }
                        }
                    }
                }
                async_wait_pending<0>();  // the ring is reused by the second sweep
            }
            Vec<4> o0, o1, o2, o3;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o0.v[k] = m[k].ar; o1.v[k] = m[k].ai; o2.v[k] = m[k].br; o3.v[k] = m[k].bi;
            }
            vec_store<4>(sum_at(smem, warp, 0) + lane * 4, o0);
            vec_store<4>(sum_at(smem, warp, 1) + lane * 4, o1);
            vec_store<4>(sum_at(smem, warp, 2) + lane * 4, o2);
            vec_store<4>(sum_at(smem, warp, 3) + lane * 4, o3);
        } else if constexpr (PH == 1) {
            if (thread < kGroup && tl.cg * kGroup + thread < C && tl.n > 0) {
                Affine a = affine_identity();
#pragma unroll
                for (int w = 0; w < WARPS; ++w)
                    a = affine_then(a, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                    sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
                publish4(p.agg + ((size_t)tl.idx * kGroup + thread) * 4, a.ar, a.ai, a.br, a.bi);
            }
        } else if constexpr (PH == 2) {
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                float sr, si;
                if (tl.n == 0) {
                    sr = p.state_in ? p.state_in[(size_t)tl.b * 2 * C + ch] : 0.0f;
                    si = p.state_in ? p.state_in[(size_t)tl.b * 2 * C + C + ch] : 0.0f;
                } else {
                    look_back(p.agg, p.incl, tl.chain * s.NT, tl.n, thread, p.ctrl, s.max_polls, sr, si);
                }
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    carry_at(smem, w, 0)[thread] = sr;
                    carry_at(smem, w, 1)[thread] = si;
                    affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                        sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                                 sr, si);
                }
                publish2(p.incl + ((size_t)tl.idx * kGroup + thread) * 2, sr, si);
                if (p.state_out && tl.n == s.NT - 1) {
                    p.state_out[(size_t)tl.b * 2 * C + ch] = sr;
                    p.state_out[(size_t)tl.b * 2 * C + C + ch] = si;
                }
            }
        } else {  // PH == 3
            if (!chan_ok) return;
            const Vec<4> lr = vec_load<4>(p.tr + c0);
            const Vec<4> li = vec_load<4>(p.ti + c0);
            const Vec<4> gm = vec_load<4>(p.gamma + c0);
            Vec<4> sr = vec_load<4>(carry_at(smem, warp, 0) + lane * 4);
            Vec<4> si = vec_load<4>(carry_at(smem, warp, 1) + lane * 4);
            IO* obase = p.read + ((size_t)tl.b * s.L) * 4 * C + c0;
#pragma unroll
            for (int j = 0; j < STAGES - 1; ++j) issue(tbeg + j * U, j);
            int stage = 0;
            for (int t0 = tbeg; t0 < tend; t0 += U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                issue(t0 + (STAGES - 1) * U, stage == 0 ? STAGES - 1 : stage - 1);
                async_wait_pending<STAGES - 1>();
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t0 + u < tend) {
                        const Vec<4> zr = cell_load4<IO>(cell_at(smem, stage, u * 3 + 0, thread));
                        const Vec<4> zi = cell_load4<IO>(cell_at(smem, stage, u * 3 + 1, thread));
                        const Vec<4> zv = cell_load4<IO>(cell_at(smem, stage, u * 3 + 2, thread));
                        Vec<4> dr, di;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const Gate g = make_gate(zr.v[k], zi.v[k], zv.v[k]);
                            float mr, mi;
                            cmul(lr.v[k], li.v[k], sr.v[k], si.v[k], mr, mi);
                            dr.v[k] = g.vac * mr;
                            di.v[k] = g.vac * mi;
                            const float bs = gm.v[k] * g.vac;
                            sr.v[k] = (1.0f - g.vac) * mr + bs * g.inj_r;
                            si.v[k] = (1.0f - g.vac) * mi + bs * g.inj_i;
                        }
                        IO* orow = obase + (size_t)(t0 + u) * 4 * C;
                        io_store4_stream(orow, sr);
                        io_store4_stream(orow + C, si);
                        io_store4_stream(orow + 2 * C, dr);
                        io_store4_stream(orow + 3 * C, di);
                    }
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------
// Backward, single pass over HBM in two sweeps per tile.
//
// The dual recurrence runs from the last step to the first, so tiles are handed out
// from the end of the sequence and "earlier in scan order" means later in time.
// Per block (WARPS warps, warp w owns TS consecutive steps):
//   sweep 1  walk the warp's steps backwards reading z_v and grad_read (5 planes) and
//            compose the warp's dual map (P, Q)            (reference :655-705);
//   publish the tile's map, look back over later-in-time tiles for the gradient carry
//            entering this tile, publish this tile's outgoing carry;
//   sweep 2  walk the same steps again from the warp's carry: the 5 planes come back
//            from L2 (the tile was read microseconds ago), z_r, z_i and s_{t-1} (from
//            the saved forward output) come from HBM; write grad_raw and accumulate
//            d lambda_r, d lambda_i, d gamma            (reference :794-909);
//   reduce the warps' parameter-gradient partials in a fixed order into one row per
//            tile; BwdReduce adds the rows.
// HBM traffic per channel-step: 20 B (sweep 1) + 16 B (z_r, z_i, s_{t-1}) + 12 B written.
// ---------------------------------------------------------------------------
// One step of the dual recurrence on two channels, composed onto the map of the later
// steps: carry_{t-1} = conj(lambda) (keep (u + carry_t) + v gd)          (reference :655-705).
// `nli` is -Im lambda.
FL_HD void dual_step2(Affine2& m, const F2& zv, const F2& ur, const F2& ui, const F2& gr,
                      const F2& gi, const F2& lr, const F2& li, const F2& nli) {
    const F2 sig = sigmoid2(zv);
    const F2 vac = mul2(sig, splat2(kVacMax));
    const F2 keep = fma2(sig, splat2(-kVacMax), splat2(1.0f));
    const F2 hr = fma2(keep, ur, mul2(vac, gr));
    const F2 hi = fma2(keep, ui, mul2(vac, gi));
    // q = conj(lambda) h;  alpha = keep conj(lambda) = (ar, na), pa = -na
    const F2 qr = fma2(lr, hr, mul2(li, hi));
    const F2 qi = fma2(lr, hi, mul2(nli, hr));
    const F2 ar = mul2(keep, lr), pa = mul2(keep, li), na = mul2(keep, nli);
    Affine2 o;
    o.br = fma2(ar, m.br, fma2(pa, m.bi, qr));
    o.bi = fma2(ar, m.bi, fma2(na, m.br, qi));
    o.ar = fma2(ar, m.ar, mul2(pa, m.ai));
    o.ai = fma2(ar, m.ai, mul2(na, m.ar));
    m = o;
}

// dual_step2 in forward time order, together with the state recurrence it shares gates with:
// advances (sr, si) from s_{t-1} to s_t = keep lambda s_{t-1} + gamma v inj and composes the
// dual step BEFORE the map of the earlier steps (the map takes the carry after step t to the
// carry before the first step).
FL_HD void recompute_step2(Affine2& m, F2& sr, F2& si, const F2& zr, const F2& zi, const F2& zv,
                           const F2& ur, const F2& ui, const F2& gr, const F2& gi, const F2& lr,
                           const F2& li, const F2& nli, const F2& gm) {
    const Gate2 g = make_gate2(zr, zi, zv);
    const F2 ar = mul2(g.keep, lr), pa = mul2(g.keep, li), na = mul2(g.keep, nli);
    const F2 bs = mul2(gm, g.vac);
    const F2 nr = fma2(ar, sr, fma2(na, si, mul2(bs, g.inj_r)));
    const F2 ni = fma2(ar, si, fma2(pa, sr, mul2(bs, g.inj_i)));
    sr = nr;
    si = ni;
    const F2 hr = fma2(g.keep, ur, mul2(g.vac, gr));
    const F2 hi = fma2(g.keep, ui, mul2(g.vac, gi));
    const F2 qr = fma2(lr, hr, mul2(li, hi));
    const F2 qi = fma2(lr, hi, mul2(nli, hr));
    // first the step (alpha = (ar, na), q), then m:  A' = A alpha,  B' = A q + B
    Affine2 o;
    o.br = fma2(m.ar, qr, fma2(mul2(m.ai, splat2(-1.0f)), qi, m.br));
    o.bi = fma2(m.ar, qi, fma2(m.ai, qr, m.bi));
    o.ar = fma2(m.ar, ar, mul2(m.ai, pa));
    o.ai = fma2(m.ar, na, mul2(m.ai, ar));
    m = o;
}

// Parameter-gradient partial sums of two channels (Im d lambda = dtia - dtib).
struct BwdAcc2 {
    F2 dtr, dtia, dtib, dgm;
};

// One step of the second backward sweep on two channels (reference :794-909): from the
// carry (cr, ci) entering step t and the saved s_{t-1} = (sr, si), the three gradients of
// the step's raw inputs, the parameter-gradient terms, and the carry leaving the step.
FL_HD void bwd_step2(const F2& zr, const F2& zi, const F2& zv, const F2& ur, const F2& ui,
                     const F2& gdr, const F2& gdi, const F2& sr, const F2& si, const F2& lr,
                     const F2& li, const F2& nli, const F2& gm, F2& cr, F2& ci, BwdAcc2& acc,
                     F2& ozr, F2& ozi, F2& ozv) {
    const F2 one = splat2(1.0f), mone = splat2(-1.0f), two = splat2(2.0f);
    const Gate2 g = make_gate2(zr, zi, zv);
    const F2 Gr = add2(ur, cr), Gi = add2(ui, ci);
    // m = lambda s_prev;  H = keep G + v gd
    const F2 mr = fma2(lr, sr, mul2(nli, si));
    const F2 mi = fma2(lr, si, mul2(li, sr));
    const F2 Hr = fma2(g.keep, Gr, mul2(g.vac, gdr));
    const F2 Hi = fma2(g.keep, Gi, mul2(g.vac, gdi));
    // d lambda += conj(s_prev) H
    acc.dtr = fma2(sr, Hr, fma2(si, Hi, acc.dtr));
    acc.dtia = fma2(sr, Hi, acc.dtia);
    acc.dtib = fma2(si, Hr, acc.dtib);
    // d gamma += v (inj . G)
    const F2 common = fma2(g.inj_r, Gr, mul2(g.inj_i, Gi));
    acc.dgm = fma2(g.vac, common, acc.dgm);
    // dv = G . (gamma inj - m) + gd . m = gamma (inj . G) + m . (gd - G)
    const F2 er = fma2(Gr, mone, gdr), ei = fma2(Gi, mone, gdi);
    const F2 dv = fma2(gm, common, fma2(mr, er, mul2(mi, ei)));
    const F2 bs = mul2(gm, g.vac);
    // 1 - tanh^2 = tanh (-tanh) + 1 with -tanh = 2 r - 1
    const F2 sech_r = fma2(g.inj_r, fma2(g.rr, two, mone), one);
    const F2 sech_i = fma2(g.inj_i, fma2(g.ri, two, mone), one);
    ozr = mul2(mul2(bs, Gr), sech_r);
    ozi = mul2(mul2(bs, Gi), sech_i);
    // v (1 - sig)
    ozv = mul2(mul2(dv, g.vac), fma2(g.sig, mone, one));
    // carry <- conj(lambda) H
    cr = fma2(lr, Hr, mul2(li, Hi));
    ci = fma2(lr, Hi, mul2(nli, Hr));
}

template <typename IO>
struct SpBwdParamsT {
    const IO* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;        // [B, 2C] or null
    const IO* read;               // saved forward output
    const IO* grad_read;
    const float* grad_state_out;  // [B, 2C] or null
    IO* grad_raw;
    float* grad_state_in;         // [B, 2C] or null
    float* agg;                   // [tiles][128][4]
    float* incl;                  // [tiles][128][2]
    unsigned* ctrl;               // error word
    float* partial;               // [3][B][NT][C]
    SpShape s;
    // Optional replacement for `read` in the kernels that recompute the states: row j holds the
    // state after step kStateRowEvery * (j + 1) - 1, [B, state_rows, 2C] fp32. Null: use `read`.
    const float* states = nullptr;
    int state_rows = 0;
};
using SpBwdParams = SpBwdParamsT<float>;
constexpr int kStateRowEvery = 8;

template <int TS, int WARPS, int U1_, int U2_, int MIN_BLOCKS, bool ASYNC = false, int STAGES = 2,
          typename IO = float>
struct BwdSinglePass {
    using Params = SpBwdParamsT<IO>;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kPhases = 5;
    static constexpr int kSplitPhase = 2;
    static constexpr int kSumFloats = WARPS * 4 * kGroup;   // warp maps, later warp partials
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;
    // ASYNC: every thread lands its next batches of inputs in a private ring of STAGES slots in shared
    // memory with cp.async while it computes on the current batch, so loads stay in flight
    // without holding registers. A cell is four elements of one thread: 16 bytes of float, 8 of
    // bfloat16 (packed, so a warp's cells of one plane are contiguous in both cases).
    static constexpr int kCellFloats = (int)sizeof(IO);
    static constexpr int kCells = U1_ * 5 > U2_ * 9 ? U1_ * 5 : U2_ * 9;
    static constexpr int kRingFloats = ASYNC ? STAGES * kCells * 32 * WARPS * kCellFloats : 0;
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kRingFloats;
    static constexpr int kClaimAfter = 2;
    FL_HD static constexpr bool barrier_after(int ph) { return ph != 1; }
    static constexpr int U1 = U1_;  // steps loaded together in sweep 1
    static constexpr int U2 = U2_;  // steps loaded together in sweep 2
    static_assert(kThreads >= kGroup, "one thread per channel is needed for the look-back");
    static_assert(TS % U1 == 0 && TS % U2 == 0, "sub-chunk must be a multiple of the unroll");

    struct State {};  // nothing lives in registers across barriers

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }
    FL_HD static float* cell_at(float* smem, int stage, int idx, int thread) {
        return smem + kSumFloats + kCarryFloats +
               ((size_t)(stage * kCells + idx) * kThreads + thread) * kCellFloats;
    }
    // Warms L2 with the first-sweep inputs (z_v, grad_read) of the tile this block takes next.
    FL_HD static void prefetch(const Params& p, int tile, int thread) {
        const SpShape& s = p.s;
        const SpTile nx = sp_decode(s, (unsigned)tile);
        const int t_lo = (s.NT - 1 - nx.n) * kTile;
        const int width = s.C - nx.cg * kGroup;
        prefetch_rows(p.raw + ((size_t)nx.b * s.L + t_lo) * 3 * s.C + 2 * s.C + nx.cg * kGroup, kTile,
                      s.L - t_lo, 1, (size_t)3 * s.C, (size_t)s.C, width, thread, kThreads);
        prefetch_rows(p.grad_read + ((size_t)nx.b * s.L + t_lo) * 4 * s.C + nx.cg * kGroup, kTile,
                      s.L - t_lo, 4, (size_t)4 * s.C, (size_t)s.C, width, thread, kThreads);
    }

    template <int PH>
    FL_HD static void phase(const Params& p, int block, int thread, float* smem, State&) {
        const SpShape& s = p.s;
        // tl.n is the position in scan order; the tile covers time tile NT-1-n
        const SpTile tl = sp_decode(s, (unsigned)block);
        const int time_tile = s.NT - 1 - tl.n;
        const int lane = thread & 31, warp = thread >> 5;
        const int slot = WARPS - 1 - warp;  // position of this warp's steps in scan order
        const int C = s.C;
        const int c0 = tl.cg * kGroup + lane * 4;
        const bool chan_ok = c0 < C;
        const int tbeg = time_tile * kTile + warp * TS;           // first step of the warp
        const int tend = tbeg + TS < s.L ? tbeg + TS : s.L;       // one past its last valid step

        if constexpr (PH == 0) {
            // Second-sweep inputs of this tile that the first sweep does not touch (z_r, z_i and
            // the previous states): start them towards L2 now, they are needed after the look-back.
            if (s.prefetch > 0) {
                const int t_lo = time_tile * kTile;
                const int width = C - tl.cg * kGroup;
                prefetch_rows(p.raw + ((size_t)tl.b * s.L + t_lo) * 3 * C + tl.cg * kGroup, kTile,
                              s.L - t_lo, 2, (size_t)3 * C, (size_t)C, width, thread, kThreads);
                const int first = t_lo > 0 ? t_lo - 1 : 0;  // row of s_{t-1} for the tile's first step
                prefetch_rows(p.read + ((size_t)tl.b * s.L + first) * 4 * C + tl.cg * kGroup, kTile,
                              s.L - 1 - first, 2, (size_t)4 * C, (size_t)C, width, thread, kThreads);
            }
            Affine2 m[2] = {affine2_identity(), affine2_identity()};
            if (chan_ok) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const IO* zbase = p.raw + ((size_t)tl.b * s.L) * 3 * C + 2 * C + c0;
                const IO* gbase = p.grad_read + ((size_t)tl.b * s.L) * 4 * C + c0;
                // Running row pointers of the next batch to issue (rows descend; the pointers may
                // step below the tile after the last batch and are not dereferenced then).
                int t_issue = tend;
                const IO* zq = zbase + (ptrdiff_t)(tend - 1) * 3 * C;
                const IO* gq = gbase + (ptrdiff_t)(tend - 1) * 4 * C;
                // batch of U1 steps ending just before t_issue, into ring slot `stage`
                auto issue1 = [&](int, int stage) {
#pragma unroll
                    for (int u = 0; u < U1; ++u) {
                        if (t_issue - 1 - u >= tbeg) {
                            const IO* grow = gq - (ptrdiff_t)u * 4 * C;
                            async_copy4(cell_at(smem, stage, u * 5 + 0, thread), zq - (ptrdiff_t)u * 3 * C);
                            async_copy4(cell_at(smem, stage, u * 5 + 1, thread), grow);
                            async_copy4(cell_at(smem, stage, u * 5 + 2, thread), grow + C);
                            async_copy4(cell_at(smem, stage, u * 5 + 3, thread), grow + 2 * C);
                            async_copy4(cell_at(smem, stage, u * 5 + 4, thread), grow + 3 * C);
                        }
                    }
                    t_issue -= U1;
                    zq -= (ptrdiff_t)U1 * 3 * C;
                    gq -= (ptrdiff_t)U1 * 4 * C;
                    async_commit();
                };
                if constexpr (ASYNC) {
#pragma unroll
                    for (int j = 0; j < STAGES - 1; ++j) issue1(tend - j * U1, j);  // empty past tbeg
                }
                int stage = 0;
                for (int t0 = tend; t0 > tbeg; t0 -= U1, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                    Vec<4> zv[U1], ur[U1], ui[U1], gr[U1], gi[U1];
                    if constexpr (ASYNC) {
                        issue1(t0 - (STAGES - 1) * U1, stage == 0 ? STAGES - 1 : stage - 1);
                        async_wait_pending<STAGES - 1>();
#pragma unroll
                        for (int u = 0; u < U1; ++u) {
                            if (t0 - 1 - u >= tbeg) {
                                zv[u] = cell_load4<IO>(cell_at(smem, stage, u * 5 + 0, thread));
                                ur[u] = cell_load4<IO>(cell_at(smem, stage, u * 5 + 1, thread));
                                ui[u] = cell_load4<IO>(cell_at(smem, stage, u * 5 + 2, thread));
                                gr[u] = cell_load4<IO>(cell_at(smem, stage, u * 5 + 3, thread));
                                gi[u] = cell_load4<IO>(cell_at(smem, stage, u * 5 + 4, thread));
                            }
                        }
                    } else {
#pragma unroll
                    for (int u = 0; u < U1; ++u) {
                        const int t = t0 - 1 - u;
                        if (t >= tbeg) {
                            zv[u] = io_load4(zbase + (size_t)t * 3 * C);
                            const IO* grow = gbase + (size_t)t * 4 * C;
                            ur[u] = io_load4(grow);
                            ui[u] = io_load4(grow + C);
                            gr[u] = io_load4(grow + 2 * C);
                            gi[u] = io_load4(grow + 3 * C);
                        }
                    }
                    }
#pragma unroll
                    for (int u = 0; u < U1; ++u) {
                        if (t0 - 1 - u >= tbeg) {
                            dual_step2(m[0], lo2(zv[u]), lo2(ur[u]), lo2(ui[u]), lo2(gr[u]), lo2(gi[u]),
                                       lr2[0], li2[0], nli2[0]);
                            dual_step2(m[1], hi2(zv[u]), hi2(ur[u]), hi2(ui[u]), hi2(gr[u]), hi2(gi[u]),
                                       lr2[1], li2[1], nli2[1]);
                        }
                    }
                }
            }
            vec_store<4>(sum_at(smem, slot, 0) + lane * 4, join2(m[0].ar, m[1].ar));
            vec_store<4>(sum_at(smem, slot, 1) + lane * 4, join2(m[0].ai, m[1].ai));
            vec_store<4>(sum_at(smem, slot, 2) + lane * 4, join2(m[0].br, m[1].br));
            vec_store<4>(sum_at(smem, slot, 3) + lane * 4, join2(m[0].bi, m[1].bi));
        } else if constexpr (PH == 1) {
            if (thread < kGroup && tl.cg * kGroup + thread < C && tl.n > 0) {
                Affine a = affine_identity();
#pragma unroll
                for (int w = 0; w < WARPS; ++w)
                    a = affine_then(a, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                    sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
                publish4(p.agg + ((size_t)tl.idx * kGroup + thread) * 4, a.ar, a.ai, a.br, a.bi);
            }
        } else if constexpr (PH == 2) {
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                float sr, si;
                if (tl.n == 0) {
                    sr = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + ch] : 0.0f;
                    si = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + C + ch] : 0.0f;
                } else {
                    look_back(p.agg, p.incl, tl.chain * s.NT, tl.n, thread, p.ctrl, s.max_polls, sr, si);
                }
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    carry_at(smem, w, 0)[thread] = sr;
                    carry_at(smem, w, 1)[thread] = si;
                    affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                        sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                                 sr, si);
                }
                publish2(p.incl + ((size_t)tl.idx * kGroup + thread) * 2, sr, si);
                if (p.grad_state_in && tl.n == s.NT - 1) {
                    p.grad_state_in[(size_t)tl.b * 2 * C + ch] = sr;
                    p.grad_state_in[(size_t)tl.b * 2 * C + C + ch] = si;
                }
            }
        } else if constexpr (PH == 3) {
            const F2 zero2 = splat2(0.0f);
            BwdAcc2 acc[2] = {{zero2, zero2, zero2, zero2}, {zero2, zero2, zero2, zero2}};
            if (chan_ok) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const F2 gm2[2] = {lo2(gm), hi2(gm)};
                const Vec<4> cr4 = vec_load<4>(carry_at(smem, slot, 0) + lane * 4);
                const Vec<4> ci4 = vec_load<4>(carry_at(smem, slot, 1) + lane * 4);
                F2 cr[2] = {lo2(cr4), hi2(cr4)}, ci[2] = {lo2(ci4), hi2(ci4)};
                const IO* zbase = p.raw + ((size_t)tl.b * s.L) * 3 * C + c0;
                const IO* gbase = p.grad_read + ((size_t)tl.b * s.L) * 4 * C + c0;
                const IO* rbase = p.read + ((size_t)tl.b * s.L) * 4 * C + c0;
                IO* obase = p.grad_raw + ((size_t)tl.b * s.L) * 3 * C + c0;
                int t_issue = tend;
                const IO* zq = zbase + (ptrdiff_t)(tend - 1) * 3 * C;
                const IO* gq = gbase + (ptrdiff_t)(tend - 1) * 4 * C;
                const IO* rq = rbase + (ptrdiff_t)(tend - 2) * 4 * C;  // row of s_{t-1}
                auto issue2 = [&](int, int stage) {
#pragma unroll
                    for (int u = 0; u < U2; ++u) {
                        const int t = t_issue - 1 - u;
                        if (t >= tbeg) {
                            const IO* zrow = zq - (ptrdiff_t)u * 3 * C;
                            const IO* grow = gq - (ptrdiff_t)u * 4 * C;
                            async_copy4(cell_at(smem, stage, u * 9 + 0, thread), zrow);
                            async_copy4(cell_at(smem, stage, u * 9 + 1, thread), zrow + C);
                            async_copy4(cell_at(smem, stage, u * 9 + 2, thread), zrow + 2 * C);
                            async_copy4(cell_at(smem, stage, u * 9 + 3, thread), grow);
                            async_copy4(cell_at(smem, stage, u * 9 + 4, thread), grow + C);
                            async_copy4(cell_at(smem, stage, u * 9 + 5, thread), grow + 2 * C);
                            async_copy4(cell_at(smem, stage, u * 9 + 6, thread), grow + 3 * C);
                            if (t > 0) {
                                const IO* prow = rq - (ptrdiff_t)u * 4 * C;
                                async_copy4(cell_at(smem, stage, u * 9 + 7, thread), prow);
                                async_copy4(cell_at(smem, stage, u * 9 + 8, thread), prow + C);
                            }
                        }
                    }
                    t_issue -= U2;
                    zq -= (ptrdiff_t)U2 * 3 * C;
                    gq -= (ptrdiff_t)U2 * 4 * C;
                    rq -= (ptrdiff_t)U2 * 4 * C;
                    async_commit();
                };
                if constexpr (ASYNC) {
#pragma unroll
                    for (int j = 0; j < STAGES - 1; ++j) issue2(tend - j * U2, j);
                }
                int stage = 0;
                for (int t0 = tend; t0 > tbeg; t0 -= U2, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                    Vec<4> zr[U2], zi[U2], zv[U2], ur[U2], ui[U2], gr[U2], gi[U2], pr[U2], pi[U2];
                    if constexpr (ASYNC) {
                        issue2(t0 - (STAGES - 1) * U2, stage == 0 ? STAGES - 1 : stage - 1);
                        async_wait_pending<STAGES - 1>();
#pragma unroll
                        for (int u = 0; u < U2; ++u) {
                            const int t = t0 - 1 - u;
                            if (t >= tbeg) {
                                zr[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 0, thread));
                                zi[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 1, thread));
                                zv[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 2, thread));
                                ur[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 3, thread));
                                ui[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 4, thread));
                                gr[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 5, thread));
                                gi[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 6, thread));
                                if (t > 0) {
                                    pr[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 7, thread));
                                    pi[u] = cell_load4<IO>(cell_at(smem, stage, u * 9 + 8, thread));
                                } else if (p.state_in) {
                                    const float* prow = p.state_in + (size_t)tl.b * 2 * C + c0;
                                    pr[u] = vec_load<4>(prow);
                                    pi[u] = vec_load<4>(prow + C);
                                } else {
                                    pr[u] = vec_fill<4>(0.0f);
                                    pi[u] = vec_fill<4>(0.0f);
                                }
                            }
                        }
                    } else {
#pragma unroll
                    for (int u = 0; u < U2; ++u) {
                        const int t = t0 - 1 - u;
                        if (t >= tbeg) {
                            const IO* zrow = zbase + (size_t)t * 3 * C;
                            zr[u] = io_load4_stream(zrow);
                            zi[u] = io_load4_stream(zrow + C);
                            zv[u] = io_load4_stream(zrow + 2 * C);
                            const IO* grow = gbase + (size_t)t * 4 * C;
                            ur[u] = io_load4_stream(grow);
                            ui[u] = io_load4_stream(grow + C);
                            gr[u] = io_load4_stream(grow + 2 * C);
                            gi[u] = io_load4_stream(grow + 3 * C);
                            if (t > 0) {
                                const IO* prow = rbase + (size_t)(t - 1) * 4 * C;
                                pr[u] = io_load4_stream(prow);
                                pi[u] = io_load4_stream(prow + C);
                            } else if (p.state_in) {
                                const float* prow = p.state_in + (size_t)tl.b * 2 * C + c0;
                                pr[u] = vec_load<4>(prow);
                                pi[u] = vec_load<4>(prow + C);
                            } else {
                                pr[u] = vec_fill<4>(0.0f);
                                pi[u] = vec_fill<4>(0.0f);
                            }
                        }
                    }
                    }
#pragma unroll
                    for (int u = 0; u < U2; ++u) {
                        const int t = t0 - 1 - u;
                        if (t >= tbeg) {
                            F2 ozr[2], ozi[2], ozv[2];
                            bwd_step2(lo2(zr[u]), lo2(zi[u]), lo2(zv[u]), lo2(ur[u]), lo2(ui[u]),
                                      lo2(gr[u]), lo2(gi[u]), lo2(pr[u]), lo2(pi[u]), lr2[0], li2[0],
                                      nli2[0], gm2[0], cr[0], ci[0], acc[0], ozr[0], ozi[0], ozv[0]);
                            bwd_step2(hi2(zr[u]), hi2(zi[u]), hi2(zv[u]), hi2(ur[u]), hi2(ui[u]),
                                      hi2(gr[u]), hi2(gi[u]), hi2(pr[u]), hi2(pi[u]), lr2[1], li2[1],
                                      nli2[1], gm2[1], cr[1], ci[1], acc[1], ozr[1], ozi[1], ozv[1]);
                            IO* orow = obase + (size_t)t * 3 * C;
                            io_store4_stream(orow, join2(ozr[0], ozr[1]));
                            io_store4_stream(orow + C, join2(ozi[0], ozi[1]));
                            io_store4_stream(orow + 2 * C, join2(ozv[0], ozv[1]));
                        }
                    }
                }
            }
            // warp partials into the (now free) map area: [warp][3][128]
            const F2 mone = splat2(-1.0f);
            vec_store<4>(sum_at(smem, warp, 0) + lane * 4, join2(acc[0].dtr, acc[1].dtr));
            vec_store<4>(sum_at(smem, warp, 1) + lane * 4,
                         join2(fma2(acc[0].dtib, mone, acc[0].dtia), fma2(acc[1].dtib, mone, acc[1].dtia)));
            vec_store<4>(sum_at(smem, warp, 2) + lane * 4, join2(acc[0].dgm, acc[1].dgm));
        } else {  // PH == 4: one partial row per tile, warps added in a fixed order
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                const size_t plane = (size_t)s.B * s.NT * C;
                float* out = p.partial + ((size_t)tl.b * s.NT + time_tile) * C + ch;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    float acc = 0.0f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) acc += sum_at(smem, w, k)[thread];
                    out[k * plane] = acc;
                }
            }
        }
    }
};


// ---------------------------------------------------------------------------
// Backward with recomputed states. Same tiles, maps, look-back and outputs as
// BwdSinglePass, but s_{t-1} is not read back from the saved forward output for every
// step. Sweep 1 walks the warp's steps FORWARD in time: it reads all seven input planes
// (z_r, z_i, z_v, grad_read), re-runs the state recurrence from the one saved row just
// before the warp's first step, parks s_{t-1} of every step in shared memory (two 16-byte
// cells per thread and step) and composes the dual map in the same pass. Sweep 2 walks
// backwards as before; its seven planes come back from L2 and s_{t-1} from shared memory.
// HBM traffic per channel-step: 28 B read + 8/TS B (the saved row) + 12 B written, which is
// the compulsory traffic of the backward plus one row per TS steps.
// ---------------------------------------------------------------------------
template <int TS, int WARPS, int U_, int MIN_BLOCKS, int STAGES, typename IO = float>
struct BwdRecompute {
    using Params = SpBwdParamsT<IO>;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kPhases = 5;
    static constexpr int kSplitPhase = 2;
    static constexpr int U = U_;  // steps per ring slot
    static constexpr int kSumFloats = WARPS * 4 * kGroup;
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;
    static constexpr int kCells = U * 7;
    static constexpr int kRingFloats = STAGES * kCells * kThreads * 4;
    static constexpr int kStashFloats = TS * 2 * kThreads * 4;
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kRingFloats + kStashFloats;
    static constexpr int kClaimAfter = 2;
    FL_HD static constexpr bool barrier_after(int ph) { return ph != 1; }
    static_assert(kThreads >= kGroup, "one thread per channel is needed for the look-back");
    static_assert(TS % U == 0, "sub-chunk must be a multiple of the unroll");

    struct State {};

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }
    FL_HD static float* cell_at(float* smem, int stage, int idx, int thread) {
        return smem + kSumFloats + kCarryFloats +
               ((size_t)(stage * kCells + idx) * kThreads + thread) * 4;
    }
    // s_{t-1} of the warp's step j (k = 0: real parts, 1: imaginary parts)
    FL_HD static float* stash_at(float* smem, int j, int k, int thread) {
        return smem + kSumFloats + kCarryFloats + kRingFloats +
               ((size_t)(j * 2 + k) * kThreads + thread) * 4;
    }
    FL_HD static void prefetch(const Params&, int, int) {}

    // the seven planes of step row (zrow, grow) into the cells of sub-step u of a slot
    FL_HD static void issue_step(float* smem, int stage, int u, int thread, const IO* zrow,
                                 const IO* grow, int C) {
        async_copy4(cell_at(smem, stage, u * 7 + 0, thread), zrow);
        async_copy4(cell_at(smem, stage, u * 7 + 1, thread), zrow + C);
        async_copy4(cell_at(smem, stage, u * 7 + 2, thread), zrow + 2 * C);
        async_copy4(cell_at(smem, stage, u * 7 + 3, thread), grow);
        async_copy4(cell_at(smem, stage, u * 7 + 4, thread), grow + C);
        async_copy4(cell_at(smem, stage, u * 7 + 5, thread), grow + 2 * C);
        async_copy4(cell_at(smem, stage, u * 7 + 6, thread), grow + 3 * C);
    }

    template <int PH>
    FL_HD static void phase(const Params& p, int block, int thread, float* smem, State&) {
        const SpShape& s = p.s;
        const SpTile tl = sp_decode(s, (unsigned)block);
        const int time_tile = s.NT - 1 - tl.n;
        const int lane = thread & 31, warp = thread >> 5;
        const int slot = WARPS - 1 - warp;  // position of this warp's steps in scan order
        const int C = s.C;
        const int c0 = tl.cg * kGroup + lane * 4;
        const bool chan_ok = c0 < C;
        const int tbeg = time_tile * kTile + warp * TS;
        const int tend = tbeg + TS < s.L ? tbeg + TS : s.L;

        if constexpr (PH == 0) {
            Affine2 m[2] = {affine2_identity(), affine2_identity()};
            if (chan_ok && tbeg < tend) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const F2 gm2[2] = {lo2(gm), hi2(gm)};
                const IO* zq = p.raw + ((size_t)tl.b * s.L + tbeg) * 3 * C + c0;
                const IO* gq = p.grad_read + ((size_t)tl.b * s.L + tbeg) * 4 * C + c0;
                int t_issue = tbeg;
                auto issue = [&](int stage) {
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (t_issue + u < tend)
                            issue_step(smem, stage, u, thread, zq + (size_t)u * 3 * C,
                                       gq + (size_t)u * 4 * C, C);
                    t_issue += U;
                    zq += (size_t)U * 3 * C;
                    gq += (size_t)U * 4 * C;
                    async_commit();
                };
#pragma unroll
                for (int j = 0; j < STAGES - 1; ++j) issue(j);
                // the state just before the warp's first step
                Vec<4> sr4, si4;
                if (tbeg > 0 && p.states) {
                    static_assert(TS == kStateRowEvery, "one saved row per warp sub-chunk");
                    const float* prow =
                        p.states + ((size_t)tl.b * p.state_rows + tbeg / TS - 1) * 2 * C + c0;
                    sr4 = vec_load<4>(prow);
                    si4 = vec_load<4>(prow + C);
                } else if (tbeg > 0) {
                    const IO* prow = p.read + ((size_t)tl.b * s.L + tbeg - 1) * 4 * C + c0;
                    sr4 = io_load4(prow);
                    si4 = io_load4(prow + C);
                } else if (p.state_in) {
                    const float* prow = p.state_in + (size_t)tl.b * 2 * C + c0;
                    sr4 = vec_load<4>(prow);
                    si4 = vec_load<4>(prow + C);
                } else {
                    sr4 = vec_fill<4>(0.0f);
                    si4 = vec_fill<4>(0.0f);
                }
                F2 sr[2] = {lo2(sr4), hi2(sr4)}, si[2] = {lo2(si4), hi2(si4)};
                int stage = 0;
                for (int t0 = tbeg; t0 < tend; t0 += U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                    issue(stage == 0 ? STAGES - 1 : stage - 1);
                    async_wait_pending<STAGES - 1>();
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (t0 + u < tend) {
                            const Vec<4> zr = cell_load4<IO>(cell_at(smem, stage, u * 7 + 0, thread));
                            const Vec<4> zi = cell_load4<IO>(cell_at(smem, stage, u * 7 + 1, thread));
                            const Vec<4> zv = cell_load4<IO>(cell_at(smem, stage, u * 7 + 2, thread));
                            const Vec<4> ur = cell_load4<IO>(cell_at(smem, stage, u * 7 + 3, thread));
                            const Vec<4> ui = cell_load4<IO>(cell_at(smem, stage, u * 7 + 4, thread));
                            const Vec<4> gr = cell_load4<IO>(cell_at(smem, stage, u * 7 + 5, thread));
                            const Vec<4> gi = cell_load4<IO>(cell_at(smem, stage, u * 7 + 6, thread));
                            vec_store<4>(stash_at(smem, t0 + u - tbeg, 0, thread), join2(sr[0], sr[1]));
                            vec_store<4>(stash_at(smem, t0 + u - tbeg, 1, thread), join2(si[0], si[1]));
                            recompute_step2(m[0], sr[0], si[0], lo2(zr), lo2(zi), lo2(zv), lo2(ur), lo2(ui),
                                            lo2(gr), lo2(gi), lr2[0], li2[0], nli2[0], gm2[0]);
                            recompute_step2(m[1], sr[1], si[1], hi2(zr), hi2(zi), hi2(zv), hi2(ur), hi2(ui),
                                            hi2(gr), hi2(gi), lr2[1], li2[1], nli2[1], gm2[1]);
                        }
                    }
                }
            }
            vec_store<4>(sum_at(smem, slot, 0) + lane * 4, join2(m[0].ar, m[1].ar));
            vec_store<4>(sum_at(smem, slot, 1) + lane * 4, join2(m[0].ai, m[1].ai));
            vec_store<4>(sum_at(smem, slot, 2) + lane * 4, join2(m[0].br, m[1].br));
            vec_store<4>(sum_at(smem, slot, 3) + lane * 4, join2(m[0].bi, m[1].bi));
        } else if constexpr (PH == 1) {
            if (thread < kGroup && tl.cg * kGroup + thread < C && tl.n > 0) {
                Affine a = affine_identity();
#pragma unroll
                for (int w = 0; w < WARPS; ++w)
                    a = affine_then(a, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                    sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
                publish4(p.agg + ((size_t)tl.idx * kGroup + thread) * 4, a.ar, a.ai, a.br, a.bi);
            }
        } else if constexpr (PH == 2) {
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                float sr, si;
                if (tl.n == 0) {
                    sr = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + ch] : 0.0f;
                    si = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + C + ch] : 0.0f;
                } else {
                    look_back(p.agg, p.incl, tl.chain * s.NT, tl.n, thread, p.ctrl, s.max_polls, sr, si);
                }
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    carry_at(smem, w, 0)[thread] = sr;
                    carry_at(smem, w, 1)[thread] = si;
                    affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                        sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                                 sr, si);
                }
                publish2(p.incl + ((size_t)tl.idx * kGroup + thread) * 2, sr, si);
                if (p.grad_state_in && tl.n == s.NT - 1) {
                    p.grad_state_in[(size_t)tl.b * 2 * C + ch] = sr;
                    p.grad_state_in[(size_t)tl.b * 2 * C + C + ch] = si;
                }
            }
        } else if constexpr (PH == 3) {
            const F2 zero2 = splat2(0.0f);
            BwdAcc2 acc[2] = {{zero2, zero2, zero2, zero2}, {zero2, zero2, zero2, zero2}};
            if (chan_ok && tbeg < tend) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const F2 gm2[2] = {lo2(gm), hi2(gm)};
                const Vec<4> cr4 = vec_load<4>(carry_at(smem, slot, 0) + lane * 4);
                const Vec<4> ci4 = vec_load<4>(carry_at(smem, slot, 1) + lane * 4);
                F2 cr[2] = {lo2(cr4), hi2(cr4)}, ci[2] = {lo2(ci4), hi2(ci4)};
                IO* obase = p.grad_raw + ((size_t)tl.b * s.L) * 3 * C + c0;
                // rows descend; the pointers may step below the tile after the last batch
                int t_issue = tend;
                const IO* zq = p.raw + ((size_t)tl.b * s.L) * 3 * C + c0 + (ptrdiff_t)(tend - 1) * 3 * C;
                const IO* gq = p.grad_read + ((size_t)tl.b * s.L) * 4 * C + c0 + (ptrdiff_t)(tend - 1) * 4 * C;
                auto issue = [&](int stage) {
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (t_issue - 1 - u >= tbeg)
                            issue_step(smem, stage, u, thread, zq - (ptrdiff_t)u * 3 * C,
                                       gq - (ptrdiff_t)u * 4 * C, C);
                    t_issue -= U;
                    zq -= (ptrdiff_t)U * 3 * C;
                    gq -= (ptrdiff_t)U * 4 * C;
                    async_commit();
                };
#pragma unroll
                for (int j = 0; j < STAGES - 1; ++j) issue(j);
                int stage = 0;
                for (int t0 = tend; t0 > tbeg; t0 -= U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
                    issue(stage == 0 ? STAGES - 1 : stage - 1);
                    async_wait_pending<STAGES - 1>();
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int t = t0 - 1 - u;
                        if (t >= tbeg) {
                            const Vec<4> zr = cell_load4<IO>(cell_at(smem, stage, u * 7 + 0, thread));
                            const Vec<4> zi = cell_load4<IO>(cell_at(smem, stage, u * 7 + 1, thread));
                            const Vec<4> zv = cell_load4<IO>(cell_at(smem, stage, u * 7 + 2, thread));
                            const Vec<4> ur = cell_load4<IO>(cell_at(smem, stage, u * 7 + 3, thread));
                            const Vec<4> ui = cell_load4<IO>(cell_at(smem, stage, u * 7 + 4, thread));
                            const Vec<4> gr = cell_load4<IO>(cell_at(smem, stage, u * 7 + 5, thread));
                            const Vec<4> gi = cell_load4<IO>(cell_at(smem, stage, u * 7 + 6, thread));
                            const Vec<4> pr = vec_load<4>(stash_at(smem, t - tbeg, 0, thread));
                            const Vec<4> pi = vec_load<4>(stash_at(smem, t - tbeg, 1, thread));
                            F2 ozr[2], ozi[2], ozv[2];
                            bwd_step2(lo2(zr), lo2(zi), lo2(zv), lo2(ur), lo2(ui), lo2(gr), lo2(gi),
                                      lo2(pr), lo2(pi), lr2[0], li2[0], nli2[0], gm2[0], cr[0], ci[0],
                                      acc[0], ozr[0], ozi[0], ozv[0]);
                            bwd_step2(hi2(zr), hi2(zi), hi2(zv), hi2(ur), hi2(ui), hi2(gr), hi2(gi),
                                      hi2(pr), hi2(pi), lr2[1], li2[1], nli2[1], gm2[1], cr[1], ci[1],
                                      acc[1], ozr[1], ozi[1], ozv[1]);
                            IO* orow = obase + (size_t)t * 3 * C;
                            io_store4_stream(orow, join2(ozr[0], ozr[1]));
                            io_store4_stream(orow + C, join2(ozi[0], ozi[1]));
                            io_store4_stream(orow + 2 * C, join2(ozv[0], ozv[1]));
                        }
                    }
                }
            }
            const F2 mone = splat2(-1.0f);
            vec_store<4>(sum_at(smem, warp, 0) + lane * 4, join2(acc[0].dtr, acc[1].dtr));
            vec_store<4>(sum_at(smem, warp, 1) + lane * 4,
                         join2(fma2(acc[0].dtib, mone, acc[0].dtia), fma2(acc[1].dtib, mone, acc[1].dtia)));
            vec_store<4>(sum_at(smem, warp, 2) + lane * 4, join2(acc[0].dgm, acc[1].dgm));
        } else {  // PH == 4: one partial row per tile, warps added in a fixed order
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                const size_t plane = (size_t)s.B * s.NT * C;
                float* out = p.partial + ((size_t)tl.b * s.NT + time_tile) * C + ch;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    float acc = 0.0f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) acc += sum_at(smem, w, k)[thread];
                    out[k * plane] = acc;
                }
            }
        }
    }
};


// ---------------------------------------------------------------------------
// Backward with the whole tile resident in shared memory and recomputed states.
// A block issues, at its very start, the asynchronous copies of ALL seven input planes of
// its tile (one commit group per step), so a tile costs one memory latency instead of one
// per ring refill, and nothing is read twice: both sweeps work from shared memory.
//   sweep 1 (forward in time)  as soon as a step has landed: gates, the state recurrence
//            from the saved row just before the warp's first step (s_{t-1} of every step
//            stays in registers), and the dual map;
//   publish, look back, publish the carry (as in BwdSinglePass);
//   sweep 2 (backward in time) from shared memory and the registers: grad_raw and the
//            parameter-gradient partial sums.
// HBM traffic per channel-step: 28 B read + 8/TS B (saved rows) + 12 B written.
// Shared memory per block: TS * 7 cells of 16 B per thread (56 KB at TS = 4, 4 warps).
// ---------------------------------------------------------------------------
template <int TS, int WARPS, int MIN_BLOCKS, typename IO = float>
struct BwdTileResident {
    using Params = SpBwdParamsT<IO>;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kPhases = 5;
    static constexpr int kSplitPhase = 2;
    static constexpr int kSumFloats = WARPS * 4 * kGroup;
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;
    static constexpr int kCellFloats = TS * 7 * kThreads * 4;
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kCellFloats;
    static constexpr int kClaimAfter = 2;
    FL_HD static constexpr bool barrier_after(int ph) { return ph != 1; }
    static_assert(kThreads >= kGroup, "one thread per channel is needed for the look-back");
    static_assert(TS <= 8, "one copy group per step, at most eight pending");

    struct State {
        F2 sr[TS][2], si[TS][2];  // s_{t-1} of the warp's steps, two channel pairs each
    };

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }
    // plane q (0..2 raw, 3..6 grad_read) of the warp's step j
    FL_HD static float* cell_at(float* smem, int j, int q, int thread) {
        return smem + kSumFloats + kCarryFloats + ((size_t)(j * 7 + q) * kThreads + thread) * 4;
    }
    FL_HD static void prefetch(const Params&, int, int) {}

    template <int PH>
    FL_HD static void phase(const Params& p, int block, int thread, float* smem, State& st) {
        const SpShape& s = p.s;
        const SpTile tl = sp_decode(s, (unsigned)block);
        const int time_tile = s.NT - 1 - tl.n;
        const int lane = thread & 31, warp = thread >> 5;
        const int slot = WARPS - 1 - warp;  // position of this warp's steps in scan order
        const int C = s.C;
        const int c0 = tl.cg * kGroup + lane * 4;
        const bool chan_ok = c0 < C;
        const int tbeg = time_tile * kTile + warp * TS;
        const int tend = tbeg + TS < s.L ? tbeg + TS : s.L;

        if constexpr (PH == 0) {
            Affine2 m[2] = {affine2_identity(), affine2_identity()};
            if (chan_ok && tbeg < tend) {
                const IO* zrow = p.raw + ((size_t)tl.b * s.L + tbeg) * 3 * C + c0;
                const IO* grow = p.grad_read + ((size_t)tl.b * s.L + tbeg) * 4 * C + c0;
#pragma unroll
                for (int j = 0; j < TS; ++j) {
                    if (tbeg + j < tend) {
                        async_copy4(cell_at(smem, j, 0, thread), zrow);
                        async_copy4(cell_at(smem, j, 1, thread), zrow + C);
                        async_copy4(cell_at(smem, j, 2, thread), zrow + 2 * C);
                        async_copy4(cell_at(smem, j, 3, thread), grow);
                        async_copy4(cell_at(smem, j, 4, thread), grow + C);
                        async_copy4(cell_at(smem, j, 5, thread), grow + 2 * C);
                        async_copy4(cell_at(smem, j, 6, thread), grow + 3 * C);
                    }
                    async_commit();
                    zrow += (size_t)3 * C;
                    grow += (size_t)4 * C;
                }
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const F2 gm2[2] = {lo2(gm), hi2(gm)};
                // the state just before the warp's first step
                Vec<4> sr4, si4;
                if (tbeg > 0) {
                    const IO* prow = p.read + ((size_t)tl.b * s.L + tbeg - 1) * 4 * C + c0;
                    sr4 = io_load4(prow);
                    si4 = io_load4(prow + C);
                } else if (p.state_in) {
                    const float* prow = p.state_in + (size_t)tl.b * 2 * C + c0;
                    sr4 = vec_load<4>(prow);
                    si4 = vec_load<4>(prow + C);
                } else {
                    sr4 = vec_fill<4>(0.0f);
                    si4 = vec_fill<4>(0.0f);
                }
                F2 sr[2] = {lo2(sr4), hi2(sr4)}, si[2] = {lo2(si4), hi2(si4)};
#pragma unroll
                for (int j = 0; j < TS; ++j) {
                    if (tbeg + j < tend) {
                        async_wait_pending_dyn(TS - 1 - j);
                        const Vec<4> zr = cell_load4<IO>(cell_at(smem, j, 0, thread));
                        const Vec<4> zi = cell_load4<IO>(cell_at(smem, j, 1, thread));
                        const Vec<4> zv = cell_load4<IO>(cell_at(smem, j, 2, thread));
                        const Vec<4> ur = cell_load4<IO>(cell_at(smem, j, 3, thread));
                        const Vec<4> ui = cell_load4<IO>(cell_at(smem, j, 4, thread));
                        const Vec<4> gr = cell_load4<IO>(cell_at(smem, j, 5, thread));
                        const Vec<4> gi = cell_load4<IO>(cell_at(smem, j, 6, thread));
                        st.sr[j][0] = sr[0]; st.sr[j][1] = sr[1];
                        st.si[j][0] = si[0]; st.si[j][1] = si[1];
                        recompute_step2(m[0], sr[0], si[0], lo2(zr), lo2(zi), lo2(zv), lo2(ur), lo2(ui),
                                        lo2(gr), lo2(gi), lr2[0], li2[0], nli2[0], gm2[0]);
                        recompute_step2(m[1], sr[1], si[1], hi2(zr), hi2(zi), hi2(zv), hi2(ur), hi2(ui),
                                        hi2(gr), hi2(gi), lr2[1], li2[1], nli2[1], gm2[1]);
                    }
                }
            }
            vec_store<4>(sum_at(smem, slot, 0) + lane * 4, join2(m[0].ar, m[1].ar));
            vec_store<4>(sum_at(smem, slot, 1) + lane * 4, join2(m[0].ai, m[1].ai));
            vec_store<4>(sum_at(smem, slot, 2) + lane * 4, join2(m[0].br, m[1].br));
            vec_store<4>(sum_at(smem, slot, 3) + lane * 4, join2(m[0].bi, m[1].bi));
        } else if constexpr (PH == 1) {
            if (thread < kGroup && tl.cg * kGroup + thread < C && tl.n > 0) {
                Affine a = affine_identity();
#pragma unroll
                for (int w = 0; w < WARPS; ++w)
                    a = affine_then(a, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                    sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
                publish4(p.agg + ((size_t)tl.idx * kGroup + thread) * 4, a.ar, a.ai, a.br, a.bi);
            }
        } else if constexpr (PH == 2) {
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                float sr, si;
                if (tl.n == 0) {
                    sr = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + ch] : 0.0f;
                    si = p.grad_state_out ? p.grad_state_out[(size_t)tl.b * 2 * C + C + ch] : 0.0f;
                } else {
                    look_back(p.agg, p.incl, tl.chain * s.NT, tl.n, thread, p.ctrl, s.max_polls, sr, si);
                }
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    carry_at(smem, w, 0)[thread] = sr;
                    carry_at(smem, w, 1)[thread] = si;
                    affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                        sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                                 sr, si);
                }
                publish2(p.incl + ((size_t)tl.idx * kGroup + thread) * 2, sr, si);
                if (p.grad_state_in && tl.n == s.NT - 1) {
                    p.grad_state_in[(size_t)tl.b * 2 * C + ch] = sr;
                    p.grad_state_in[(size_t)tl.b * 2 * C + C + ch] = si;
                }
            }
        } else if constexpr (PH == 3) {
            const F2 zero2 = splat2(0.0f);
            BwdAcc2 acc[2] = {{zero2, zero2, zero2, zero2}, {zero2, zero2, zero2, zero2}};
            if (chan_ok && tbeg < tend) {
                const Vec<4> lr = vec_load<4>(p.tr + c0);
                const Vec<4> li = vec_load<4>(p.ti + c0);
                const Vec<4> gm = vec_load<4>(p.gamma + c0);
                const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
                const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
                const F2 gm2[2] = {lo2(gm), hi2(gm)};
                const Vec<4> cr4 = vec_load<4>(carry_at(smem, slot, 0) + lane * 4);
                const Vec<4> ci4 = vec_load<4>(carry_at(smem, slot, 1) + lane * 4);
                F2 cr[2] = {lo2(cr4), hi2(cr4)}, ci[2] = {lo2(ci4), hi2(ci4)};
                IO* obase = p.grad_raw + ((size_t)tl.b * s.L) * 3 * C + c0;
#pragma unroll
                for (int j = TS - 1; j >= 0; --j) {
                    const int t = tbeg + j;
                    if (t < tend) {
                        const Vec<4> zr = cell_load4<IO>(cell_at(smem, j, 0, thread));
                        const Vec<4> zi = cell_load4<IO>(cell_at(smem, j, 1, thread));
                        const Vec<4> zv = cell_load4<IO>(cell_at(smem, j, 2, thread));
                        const Vec<4> ur = cell_load4<IO>(cell_at(smem, j, 3, thread));
                        const Vec<4> ui = cell_load4<IO>(cell_at(smem, j, 4, thread));
                        const Vec<4> gr = cell_load4<IO>(cell_at(smem, j, 5, thread));
                        const Vec<4> gi = cell_load4<IO>(cell_at(smem, j, 6, thread));
                        F2 ozr[2], ozi[2], ozv[2];
                        bwd_step2(lo2(zr), lo2(zi), lo2(zv), lo2(ur), lo2(ui), lo2(gr), lo2(gi),
                                  st.sr[j][0], st.si[j][0], lr2[0], li2[0], nli2[0], gm2[0], cr[0], ci[0],
                                  acc[0], ozr[0], ozi[0], ozv[0]);
                        bwd_step2(hi2(zr), hi2(zi), hi2(zv), hi2(ur), hi2(ui), hi2(gr), hi2(gi),
                                  st.sr[j][1], st.si[j][1], lr2[1], li2[1], nli2[1], gm2[1], cr[1], ci[1],
                                  acc[1], ozr[1], ozi[1], ozv[1]);
                        IO* orow = obase + (size_t)t * 3 * C;
                        io_store4_stream(orow, join2(ozr[0], ozr[1]));
                        io_store4_stream(orow + C, join2(ozi[0], ozi[1]));
                        io_store4_stream(orow + 2 * C, join2(ozv[0], ozv[1]));
                    }
                }
            }
            const F2 mone = splat2(-1.0f);
            vec_store<4>(sum_at(smem, warp, 0) + lane * 4, join2(acc[0].dtr, acc[1].dtr));
            vec_store<4>(sum_at(smem, warp, 1) + lane * 4,
                         join2(fma2(acc[0].dtib, mone, acc[0].dtia), fma2(acc[1].dtib, mone, acc[1].dtia)));
            vec_store<4>(sum_at(smem, warp, 2) + lane * 4, join2(acc[0].dgm, acc[1].dgm));
        } else {  // PH == 4: one partial row per tile, warps added in a fixed order
            const int ch = tl.cg * kGroup + thread;
            if (thread < kGroup && ch < C) {
                const size_t plane = (size_t)s.B * s.NT * C;
                float* out = p.partial + ((size_t)tl.b * s.NT + time_tile) * C + ch;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    float acc = 0.0f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) acc += sum_at(smem, w, k)[thread];
                    out[k * plane] = acc;
                }
            }
        }
    }
};


// ---------------------------------------------------------------------------
// Self-test of the bounded wait: one block looks back over a chain in which nothing was
// ever published. Every thread must give up after `max_polls` polls, record the error
// word and return NaN; the kernel ends normally. Used by the tests to check, without
// hanging or faulting anything, that a lost publication turns into a status code.
// ---------------------------------------------------------------------------
struct WaitSelfTest {
    struct Params {
        const float* agg;
        const float* incl;
        unsigned* ctrl;
        float* out;  // [128][2]
        unsigned max_polls;
    };
    static constexpr int kThreads = kGroup;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int, int thread, float*) {
        float sr, si;
        look_back(p.agg, p.incl, 0, 3, thread, p.ctrl, p.max_polls, sr, si);
        p.out[thread * 2] = sr;
        p.out[thread * 2 + 1] = si;
    }
};


// ---------------------------------------------------------------------------
// Streaming chunk summary for sequence sharding: the affine map of every chunk of a span,
// reading raw once at full speed. One warp owns one (batch row, chunk, 128-channel group)
// and walks its chunk forward in batches of U steps; each thread lands the next batches in
// a private ring of STAGES slots with cp.async (3 vectors per step) while it evaluates the
// gates and composes the map of the current one. Output: the chunk maps in the layout of
// the three-phase kernels, sum [4][B][N][C], which SpanCompose folds into the span's map.
// ---------------------------------------------------------------------------
template <int U, int STAGES, int WARPS>
struct ChunkSummaryStream {
    // raw, tr, ti, gamma, sum, shape: ts = steps per warp, N = maps written per sequence
    // (one per block = WARPS consecutive warp chunks), G = 128-channel groups
    using Params = FwdParams;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kPhases = 2;
    static constexpr int kCells = U * 3;
    static constexpr int kRingFloats = STAGES * kCells * kThreads * 4;
    static constexpr int kSmemFloats = kRingFloats + WARPS * 4 * 128;  // + the warps' maps

    FL_HD static float* cell_at(float* smem, int stage, int idx, int thread) {
        return smem + ((size_t)(stage * kCells + idx) * kThreads + thread) * 4;
    }

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int lane = thread & 31, warp = thread >> 5;
        // block -> (batch row, map index, channel group); warp w takes the w-th chunk of the map
        const int cg = block % s.G;
        const int n = (block / s.G) % s.N;
        const int b = block / (s.G * s.N);
        const int C = s.C;
        const int c0 = (cg * 32 + lane) * 4;
        float* maps = smem + kRingFloats + warp * 4 * 128 + lane * 4;
        if (c0 >= C) return;
        const int t_first = (n * WARPS + warp) * s.ts;
        const int tbeg = t_first < s.L ? t_first : s.L;
        const int tend = tbeg + s.ts < s.L ? tbeg + s.ts : s.L;
        const Vec<4> lr = vec_load<4>(p.tr + c0);
        const Vec<4> li = vec_load<4>(p.ti + c0);
        const Vec<4> gm = vec_load<4>(p.gamma + c0);
        const float* base = p.raw + ((size_t)b * s.L) * 3 * C + c0;
        Affine m[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] = affine_identity();

        auto issue = [&](int t0, int stage) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 + u;
                if (t < tend) {
                    const float* row = base + (size_t)t * 3 * C;
                    async_copy16(cell_at(smem, stage, u * 3 + 0, thread), row);
                    async_copy16(cell_at(smem, stage, u * 3 + 1, thread), row + C);
                    async_copy16(cell_at(smem, stage, u * 3 + 2, thread), row + 2 * C);
                }
            }
            async_commit();
        };
#pragma unroll
        for (int j = 0; j < STAGES - 1; ++j) issue(tbeg + j * U, j);
        int stage = 0;
        for (int t0 = tbeg; t0 < tend; t0 += U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
            issue(t0 + (STAGES - 1) * U, stage == 0 ? STAGES - 1 : stage - 1);
            async_wait_pending<STAGES - 1>();
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t0 + u < tend) {
                    const Vec<4> zr = vec_load<4>(cell_at(smem, stage, u * 3 + 0, thread));
                    const Vec<4> zi = vec_load<4>(cell_at(smem, stage, u * 3 + 1, thread));
                    const Vec<4> zv = vec_load<4>(cell_at(smem, stage, u * 3 + 2, thread));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const Gate g = make_gate(zr.v[k], zi.v[k], zv.v[k]);
                        const float keep = 1.0f - g.vac;
                        const float bs = gm.v[k] * g.vac;
                        m[k] = affine_then(m[k], keep * lr.v[k], keep * li.v[k], bs * g.inj_r,
                                           bs * g.inj_i);
                    }
                }
            }
        }
        Vec<4> o0, o1, o2, o3;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o0.v[k] = m[k].ar; o1.v[k] = m[k].ai; o2.v[k] = m[k].br; o3.v[k] = m[k].bi;
        }
        vec_store<4>(maps, o0);
        vec_store<4>(maps + 128, o1);
        vec_store<4>(maps + 256, o2);
        vec_store<4>(maps + 384, o3);
    }

    // the block's map = its warps' maps in time order; one thread per channel
    FL_HD static void phase1(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int cg = block % s.G;
        const int n = (block / s.G) % s.N;
        const int b = block / (s.G * s.N);
        const int c = cg * 128 + thread;
        if (thread >= 128 || c >= s.C) return;
        Affine a = affine_identity();
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float* q = smem + kRingFloats + w * 4 * 128 + thread;
            a = affine_then(a, q[0], q[128], q[256], q[384]);
        }
        const size_t plane = (size_t)s.B * s.N * s.C;
        float* out = p.sum + ((size_t)b * s.N + n) * s.C + c;
        out[0] = a.ar; out[plane] = a.ai; out[2 * plane] = a.br; out[3 * plane] = a.bi;
    }
};


// ---------------------------------------------------------------------------
// The same for the backward pass of a sharded sequence: the dual map of every chunk of a
// span (carry before the chunk = P * carry after it + Q), reading z_v and grad_read once.
// One warp walks its chunk from its last step to its first, five vectors per step through
// the same kind of ring; the block's map composes its warps' maps, later chunks first.
// Output layout as BwdSummary: sum [4][B][N][C] = Re P | Im P | Re Q | Im Q per chunk.
// ---------------------------------------------------------------------------
template <int U, int STAGES, int WARPS>
struct ChunkDualSummaryStream {
    using Params = BwdParams;  // raw, tr, ti, grad_read, sum, s (ts, N, G as ChunkSummaryStream)
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kPhases = 2;
    static constexpr int kCells = U * 5;
    static constexpr int kRingFloats = STAGES * kCells * kThreads * 4;
    static constexpr int kSmemFloats = kRingFloats + WARPS * 4 * 128;

    FL_HD static float* cell_at(float* smem, int stage, int idx, int thread) {
        return smem + ((size_t)(stage * kCells + idx) * kThreads + thread) * 4;
    }

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int lane = thread & 31, warp = thread >> 5;
        const int cg = block % s.G;
        const int n = (block / s.G) % s.N;
        const int b = block / (s.G * s.N);
        const int C = s.C;
        const int c0 = (cg * 32 + lane) * 4;
        float* maps = smem + kRingFloats + warp * 4 * 128 + lane * 4;
        if (c0 >= C) return;
        const int t_first = (n * WARPS + warp) * s.ts;
        const int tbeg = t_first < s.L ? t_first : s.L;
        const int tend = tbeg + s.ts < s.L ? tbeg + s.ts : s.L;
        const Vec<4> lr = vec_load<4>(p.tr + c0);
        const Vec<4> li = vec_load<4>(p.ti + c0);
        const F2 lr2[2] = {lo2(lr), hi2(lr)}, li2[2] = {lo2(li), hi2(li)};
        const F2 nli2[2] = {mul2(li2[0], splat2(-1.0f)), mul2(li2[1], splat2(-1.0f))};
        const float* zbase = p.raw + ((size_t)b * s.L) * 3 * C + 2 * C + c0;
        const float* gbase = p.grad_read + ((size_t)b * s.L) * 4 * C + c0;
        Affine2 m[2] = {affine2_identity(), affine2_identity()};

        // batch of U steps ending just before t1 (rows descend), into ring slot `stage`
        auto issue = [&](int t1, int stage) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t1 - 1 - u;
                if (t >= tbeg) {
                    const float* grow = gbase + (size_t)t * 4 * C;
                    async_copy16(cell_at(smem, stage, u * 5 + 0, thread), zbase + (size_t)t * 3 * C);
                    async_copy16(cell_at(smem, stage, u * 5 + 1, thread), grow);
                    async_copy16(cell_at(smem, stage, u * 5 + 2, thread), grow + C);
                    async_copy16(cell_at(smem, stage, u * 5 + 3, thread), grow + 2 * C);
                    async_copy16(cell_at(smem, stage, u * 5 + 4, thread), grow + 3 * C);
                }
            }
            async_commit();
        };
#pragma unroll
        for (int j = 0; j < STAGES - 1; ++j) issue(tend - j * U, j);
        int stage = 0;
        for (int t1 = tend; t1 > tbeg; t1 -= U, stage = stage + 1 == STAGES ? 0 : stage + 1) {
            issue(t1 - (STAGES - 1) * U, stage == 0 ? STAGES - 1 : stage - 1);
            async_wait_pending<STAGES - 1>();
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (t1 - 1 - u >= tbeg) {
                    const Vec<4> zv = vec_load<4>(cell_at(smem, stage, u * 5 + 0, thread));
                    const Vec<4> ur = vec_load<4>(cell_at(smem, stage, u * 5 + 1, thread));
                    const Vec<4> ui = vec_load<4>(cell_at(smem, stage, u * 5 + 2, thread));
                    const Vec<4> gr = vec_load<4>(cell_at(smem, stage, u * 5 + 3, thread));
                    const Vec<4> gi = vec_load<4>(cell_at(smem, stage, u * 5 + 4, thread));
                    dual_step2(m[0], lo2(zv), lo2(ur), lo2(ui), lo2(gr), lo2(gi), lr2[0], li2[0], nli2[0]);
                    dual_step2(m[1], hi2(zv), hi2(ur), hi2(ui), hi2(gr), hi2(gi), lr2[1], li2[1], nli2[1]);
                }
            }
        }
        vec_store<4>(maps, join2(m[0].ar, m[1].ar));
        vec_store<4>(maps + 128, join2(m[0].ai, m[1].ai));
        vec_store<4>(maps + 256, join2(m[0].br, m[1].br));
        vec_store<4>(maps + 384, join2(m[0].bi, m[1].bi));
    }

    // the block's map = its warps' maps, the later chunk first; one thread per channel
    FL_HD static void phase1(const Params& p, int block, int thread, float* smem) {
        const Shape& s = p.s;
        const int cg = block % s.G;
        const int n = (block / s.G) % s.N;
        const int b = block / (s.G * s.N);
        const int c = cg * 128 + thread;
        if (thread >= 128 || c >= s.C) return;
        Affine a = affine_identity();
#pragma unroll
        for (int w = WARPS - 1; w >= 0; --w) {
            const float* q = smem + kRingFloats + w * 4 * 128 + thread;
            a = affine_then(a, q[0], q[128], q[256], q[384]);
        }
        const size_t plane = (size_t)s.B * s.N * s.C;
        float* out = p.sum + ((size_t)b * s.N + n) * s.C + c;
        out[0] = a.ar; out[plane] = a.ai; out[2 * plane] = a.br; out[3 * plane] = a.bi;
    }
};


// ---------------------------------------------------------------------------
// Exchange of span summaries between GPUs through peer memory (no collective library).
//
// Every rank owns a mailbox in memory that its peers can write:
//   mailbox [2 parities][P ranks][B][4][C] of (value, tag) pairs, 8 bytes each.
// PutSummary composes the span's map (as SpanCompose does) and stores it, tagged with the
// call's epoch, into slot [epoch & 1][rank] of EVERY rank's mailbox with plain 8-byte
// stores over NVLink: a pair is one store, so data and tag arrive together and no flag or
// fence is needed. FoldMailbox polls its own mailbox until all P slots of that parity
// carry the epoch (bounded wait), then folds the maps of the ranks before its own onto
// the initial state. Waiting for all ranks, not only the earlier ones, keeps any rank at
// most one call ahead of the slowest, so two parities are enough and nothing is ever
// cleared. Epochs are per-call counters kept by the caller, equal on all ranks, never 0.
// ---------------------------------------------------------------------------
struct MailPair { float value; unsigned tag; };

FL_HD void mail_store(MailPair* p, float value, unsigned tag) {
#if FL_DEVICE_CODE
    asm volatile("st.volatile.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(value)),
                 "r"(tag)
                 : "memory");
#else
    p->value = value;
    p->tag = tag;
#endif
}

FL_HD MailPair mail_load(const MailPair* p) {
    MailPair r;
#if FL_DEVICE_CODE
    unsigned v;
    asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];" : "=r"(v), "=r"(r.tag) : "l"(p) : "memory");
    r.value = __uint_as_float(v);
#else
    r = *p;
#endif
    return r;
}

constexpr int kMaxRanks = 16;
constexpr int kMailWindow = 4;  // ranks whose mailbox slots a waiting thread fetches together

struct PutSummary {
    struct Params {
        const float* sum;            // [4][B][N][C] chunk maps of this rank's span
        MailPair* mailbox[kMaxRanks];  // every rank's mailbox (peer pointers), index = rank
        float* summary;              // [B][4][C] local copy (may be null)
        int rank, P;
        unsigned epoch;
        Shape s;
        int reverse;                 // non-zero: the chunk maps are dual maps, composed last first
    };
    static constexpr int kThreads = 32 * kCarryWarps;
    static constexpr int kPhases = 2;
    static constexpr int kSmemFloats = 4 * kThreads;

    FL_HD static void phase0(const Params& p, int block, int thread, float* smem) {
        SpanCompose::Params q{p.sum, nullptr, p.s, p.reverse};
        SpanCompose::phase0(q, block, thread, smem);
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
        const float v[4] = {m.ar, m.ai, m.br, m.bi};
        if (p.summary) {
            float* o = p.summary + (size_t)b * 4 * s.C + c;
            for (int k = 0; k < 4; ++k) o[(size_t)k * s.C] = v[k];
        }
        const size_t slot = (((size_t)(p.epoch & 1u) * p.P + p.rank) * s.B + b) * 4 * s.C + c;
        for (int r = 0; r < p.P; ++r)
            for (int k = 0; k < 4; ++k) mail_store(p.mailbox[r] + slot + (size_t)k * s.C, v[k], p.epoch);
    }
};

struct FoldMailbox {
    struct Params {
        const MailPair* mailbox;  // this rank's own mailbox
        const float* state0;      // [B, 2C] or null
        float* state;             // [B, 2C] state entering this rank's span
        unsigned* error;          // error word (0 = ok), set to 1 if a wait ran out
        int rank, P, B, C;
        unsigned epoch, max_polls;
        int reverse;  // non-zero: fold the ranks after `rank`, last first (gradient carry)
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
        bool failed = false;
        // Four ranks' slots (16 pairs) are fetched together, so a mailbox that is already full
        // costs P / 4 round trips to L2 instead of 4 P; a slot found empty is polled on its own.
        for (int j0 = 0; j0 < p.P; j0 += kMailWindow) {
            MailPair got[kMailWindow][4];
#pragma unroll
            for (int w = 0; w < kMailWindow; ++w) {
                if (j0 + w < p.P) {
                    const int r = p.reverse ? p.P - 1 - (j0 + w) : j0 + w;
                    const MailPair* q =
                        p.mailbox + (((size_t)(p.epoch & 1u) * p.P + r) * p.B + b) * 4 * p.C + c;
#pragma unroll
                    for (int k = 0; k < 4; ++k) got[w][k] = mail_load(q + (size_t)k * p.C);
                }
            }
#pragma unroll
            for (int w = 0; w < kMailWindow; ++w) {
                if (j0 + w < p.P) {
                    const int r = p.reverse ? p.P - 1 - (j0 + w) : j0 + w;
                    const MailPair* q =
                        p.mailbox + (((size_t)(p.epoch & 1u) * p.P + r) * p.B + b) * 4 * p.C + c;
                    float v[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        MailPair m = got[w][k];
#if FL_DEVICE_CODE
                        unsigned polls = 0;
                        // a slot that is late ends the waiting for all that follow it: one bound per call
                        while (m.tag != p.epoch && !failed && ++polls < p.max_polls) {
                            backoff(polls);
                            m = mail_load(q + (size_t)k * p.C);
                        }
#endif
                        if (m.tag != p.epoch) failed = true;
                        v[k] = m.value;
                    }
                    if (p.reverse ? r > p.rank : r < p.rank)
                        affine_apply(Affine{v[0], v[1], v[2], v[3]}, sr, si);
                }
            }
        }
        if (failed) {
#if FL_DEVICE_CODE
            atomicExch(p.error, 1u);
#else
            *p.error = 1u;
#endif
            sr = si = nanf("");
        }
        p.state[(size_t)b * 2 * p.C + c] = sr;
        p.state[(size_t)b * 2 * p.C + p.C + c] = si;
    }
};

// ---------------------------------------------------------------------------
// Sum of a short vector over the ranks through the same mailboxes (the 3 C parameter-gradient
// sums of a sequence-sharded backward pass, plus the ranks' status words): every rank stores
// its n values, tagged with the call's epoch, into its slot of EVERY rank's reduction region
// (plain 8-byte peer stores), then waits with a bound until all P slots of its own region carry
// the epoch and adds them in rank order, so every rank gets the same bits. One launch, no
// collective library. Region: [2 parities][P ranks][n_max] pairs behind the mailbox's board.
// ---------------------------------------------------------------------------
struct SumMailbox {
    struct Params {
        const float* values;           // [n] this rank's addends
        float* out;                    // [n] the sum over the ranks
        MailPair* region[kMaxRanks];   // every rank's reduction region (peer pointers), index = rank
        unsigned* error;               // error word (0 = ok), set to 1 if a wait ran out
        int rank, P, n, n_max;
        unsigned epoch, max_polls;
        int stages;                    // bit 0: store, bit 1: wait and add (the host emulation runs the ranks in turn)
    };
    static constexpr int kThreads = 128;
    static constexpr int kPhases = 1;
    static constexpr int kSmemFloats = 0;

    FL_HD static void phase0(const Params& p, int block, int thread, float*) {
        const int i = block * kThreads + thread;
        if (i >= p.n) return;
        const size_t parity = (size_t)(p.epoch & 1u) * p.P;
        if (p.stages & 1) {
            const float v = p.values[i];
            for (int r = 0; r < p.P; ++r)
                mail_store(p.region[r] + (parity + p.rank) * p.n_max + i, v, p.epoch);
        }
        if (!(p.stages & 2)) return;
        const MailPair* own = p.region[p.rank];
        float acc = 0.0f;
        bool failed = false;
        for (int r0 = 0; r0 < p.P; r0 += kMailWindow) {
            MailPair got[kMailWindow];
#pragma unroll
            for (int w = 0; w < kMailWindow; ++w)
                if (r0 + w < p.P) got[w] = mail_load(own + (parity + r0 + w) * p.n_max + i);
#pragma unroll
            for (int w = 0; w < kMailWindow; ++w) {
                if (r0 + w < p.P) {
                    MailPair m = got[w];
#if FL_DEVICE_CODE
                    unsigned polls = 0;
                    while (m.tag != p.epoch && !failed && ++polls < p.max_polls) {
                        backoff(polls);
                        m = mail_load(own + (parity + r0 + w) * p.n_max + i);
                    }
#endif
                    if (m.tag != p.epoch) failed = true;
                    acc += m.value;
                }
            }
        }
        if (failed) {
#if FL_DEVICE_CODE
            atomicExch(p.error, 1u);
#else
            *p.error = 1u;
#endif
            acc = nanf("");
        }
        p.out[i] = acc;
    }
};

}  // namespace fields
