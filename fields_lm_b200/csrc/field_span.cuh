// Sequence-sharded forward in ONE launch per rank: span summary, exchange over peer memory
// and the span's forward pass, with the span read from HBM once.
//
// A sequence is cut into P contiguous spans, one per GPU. A rank needs the state entering
// its span, which is the fold of the affine maps of all earlier spans onto the initial
// state; every rank's own map needs one pass over its span. This kernel makes that pass
// and the forward pass two sweeps of the same persistent blocks:
//
//   sweep 1   the span is cut into runs (chain = batch row x 128 channels; a run = a
//             contiguous stretch of steps of one chain, one run per block when the grid
//             allows); a block walks its run from the last tile to the first, evaluates the
//             gates and composes the run's affine map (reference :493-509). Loads are
//             ordinary (cached) loads: what was read last stays in L2.
//   scan      a block stores its run's map on the rank's board and counts itself in on the
//             chain's counter, one release-acquire atomic; the last one in resets the counter
//             and writes the call's epoch into the chain's ready word. Every block waits (one
//             thread polls that word, bounded) and then composes, itself, the maps of the
//             runs before its own: the map from the span's start to the start of its run. All
//             loads are independent, two threads share a channel, so the longest chain of
//             dependent work is half the runs of a chain. The block that owns the chain's last
//             run thereby holds the span's own map and stores it into every rank's mailbox
//             over NVLink (8-byte value+tag peer stores, as PutSummary does).
//   wait      the block waits (bounded) for the summaries of all P ranks in its own mailbox,
//             folds the earlier ranks onto the initial state and applies its prefix map: the
//             state entering its run. The first tile of sweep 2 is loaded and its gates are
//             evaluated BEFORE any of this, so that work hides the scan for every block but
//             the last to finish sweep 1.
//   sweep 2   the block walks its run forward - first tile first, i.e. the rows it read
//             most recently, which a 126 MB L2 still holds when the span's raw fits
//             (8,192 tokens x 6 KB = 50 MB at 8 ranks) - and runs the recurrence, writing
//             `read` with streaming stores (reference :599-622).
//
// Blocks wait for one another (scan) and for peers (mailbox), so all blocks of the grid must
// be resident: the launch is cooperative and the grid is sized from the occupancy query.
// The board (run maps, counters, ready words) lives behind the mailbox's slots, memory zeroed
// once that only this rank's kernels touch; nothing is cleared between launches.
// Every wait is bounded; on expiry the block records the error word, poisons its state with
// NaN and finishes. Peer memory is touched by plain stores only (no TMA, no multicast).
//
// The reference has no counterpart: it runs a sequence on one GPU, and its serial carry
// kernel (:519-550) is what the scan replaces.
#pragma once

#include "field_singlepass.cuh"

namespace fields {

constexpr int kSpanMailWindow = 2;  // ranks whose slots a thread of the one-launch forward fetches together

struct SpanShape {
    int B, L, C;
    int G;          // 128-channel groups
    int chains;     // B * G
    int run_steps;  // steps per run (a multiple of the tile length)
    int R;          // runs per chain
    int items;      // chains * R; item = run * chains + chain
};

struct SpanFwdParams {
    const float* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state0;     // [B, 2C] or null: state before the FIRST span (same on every rank)
    float* read;             // [B, L, 4C]
    float* state_out;        // [B, 2C] or null: state after this rank's span
    float* summary;          // [B, 4, C] or null: this span's own map
    float* runmap;           // [items][128][4] run maps, on the rank's board
    unsigned* count;         // [chains] runs arrived (zero between launches), on the rank's board
    unsigned* ready;         // [chains] epoch of the last completed chain, 64 words apart
    int emu_round;           // host emulation: only the block's item of this round (-1: all)
    unsigned* error;         // error word (0 = ok)
    MailPair* mailbox[kMaxRanks];  // every rank's mailbox slots as seen from this GPU
    const MailPair* own;     // this rank's own slots
    int rank, P;
    unsigned epoch, max_polls;
    unsigned* epoch_word;    // null, or two words on the rank's board: [0] the epoch of the last
                             // completed call, [1] blocks of the running call that have finished.
                             // Then the kernel takes its epoch from there and the call carries none,
                             // so a captured CUDA graph can replay it.
    int stages;              // bit 0: sweep 1, bit 1: prefix, exchange and sweep 2; bit 2 (host emulation,
                             // which runs the ranks in turn): prefix and the sending half of the exchange only
    SpanShape s;
};

// CH steps per chunk (two chunks of a warp are in flight), WARPS warps, MIN_BLOCKS blocks per SM.
template <int CH, int WARPS, int MIN_BLOCKS>
struct FwdSpanSweep {
    using Params = SpanFwdParams;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = MIN_BLOCKS;
    static constexpr int kRunQuantum = WARPS;                // run lengths are multiples of this
    static constexpr int kSumFloats = WARPS * 4 * kGroup;    // the warps' maps, kept from sweep 1 to sweep 2
    static constexpr int kCarryFloats = WARPS * 2 * kGroup;  // scan: shares and prefix; then each warp's entering state
    static constexpr int kFlagFloats = 4;                    // the wait flag
    static constexpr int kSmemFloats = kSumFloats + kCarryFloats + kFlagFloats;
    static_assert(kThreads >= kGroup, "one thread per channel is needed for the carries");

    struct State {};  // nothing lives in registers across block barriers

    FL_HD static float* sum_at(float* smem, int w, int k) { return smem + (w * 4 + k) * kGroup; }
    FL_HD static float* carry_at(float* smem, int w, int k) {
        return smem + kSumFloats + (w * 2 + k) * kGroup;
    }

    struct Item {
        int chain, run, b, cg;
        int lo, hi;   // steps of the run
        int per;      // steps per warp: warp w owns [lo + w per, lo + (w + 1) per) within the run
    };
    FL_HD static Item decode(const SpanShape& s, int item) {
        Item it;
        it.chain = item % s.chains;
        it.run = item / s.chains;
        it.b = it.chain / s.G;
        it.cg = it.chain % s.G;
        it.lo = it.run * s.run_steps;
        it.hi = it.lo + s.run_steps < s.L ? it.lo + s.run_steps : s.L;
        it.per = (it.hi - it.lo + WARPS - 1) / WARPS;
        return it;
    }
    FL_HD static void warp_steps(const Item& it, int warp, int& wlo, int& whi) {
        wlo = it.lo + warp * it.per < it.hi ? it.lo + warp * it.per : it.hi;
        whi = wlo + it.per < it.hi ? wlo + it.per : it.hi;
    }

    // One chunk of a warp: CH consecutive rows of the three raw planes, four channels per lane.
    struct Chunk { Vec<4> zr[CH], zi[CH], zv[CH]; };

    // Issues the loads of rows [t0, t0 + CH) clipped to [wlo, whi) (nothing waits for them here).
    // KEEP: the rows are read again by sweep 2, so they go to L2 and stay; else evict first.
    template <bool KEEP>
    FL_HD static void chunk_load(Chunk& c, const float* base, int C, int t0, int wlo, int whi) {
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const int t = t0 + u;
            if (t >= wlo && t < whi) {
                const float* row = base + (size_t)t * 3 * C;
                if constexpr (KEEP) {
                    c.zr[u] = vec_load_l2<4>(row);
                    c.zi[u] = vec_load_l2<4>(row + C);
                    c.zv[u] = vec_load_l2<4>(row + 2 * C);
                } else {
                    c.zr[u] = vec_load_stream<4>(row);
                    c.zi[u] = vec_load_stream<4>(row + C);
                    c.zv[u] = vec_load_stream<4>(row + 2 * C);
                }
            }
        }
    }

    // The map "first the step (a, b), then m":  s -> A (a s + b) + B.
    FL_HD static Affine step_before(const Affine& m, float a_r, float a_i, float b_r, float b_i) {
        Affine o;
        o.br = m.ar * b_r - m.ai * b_i + m.br;
        o.bi = m.ar * b_i + m.ai * b_r + m.bi;
        o.ar = m.ar * a_r - m.ai * a_i;
        o.ai = m.ar * a_i + m.ai * a_r;
        return o;
    }

    // sweep 1, one chunk: the steps go in front of the warp's map so far, last row first
    FL_HD static void chunk_fold(const Chunk& c, Affine (&m)[4], const Vec<4>& lr, const Vec<4>& li,
                                 const Vec<4>& gm, int t0, int wlo, int whi) {
#pragma unroll
        for (int u = CH - 1; u >= 0; --u) {
            const int t = t0 + u;
            if (t >= wlo && t < whi) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const Gate g = make_gate(c.zr[u].v[k], c.zi[u].v[k], c.zv[u].v[k]);
                    const float keep = 1.0f - g.vac;
                    const float bs = gm.v[k] * g.vac;
                    m[k] = step_before(m[k], keep * lr.v[k], keep * li.v[k], bs * g.inj_r, bs * g.inj_i);
                }
            }
        }
    }

    // Sweep 1 of one warp: its steps from the last chunk to the first, two chunks in flight, no
    // block barrier anywhere; the warp's map goes to shared memory (reference :493-509).
    FL_HD static void sweep1_warp(const Params& p, const Item& it, int thread, float* smem) {
        const SpanShape& s = p.s;
        const int lane = thread & 31, warp = thread >> 5;
        const int C = s.C;
        const int c0 = it.cg * kGroup + lane * 4;
        Affine m[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] = affine_identity();
        int wlo, whi;
        warp_steps(it, warp, wlo, whi);
        if (c0 < C && wlo < whi) {
            const Vec<4> lr = vec_load<4>(p.tr + c0);
            const Vec<4> li = vec_load<4>(p.ti + c0);
            const Vec<4> gm = vec_load<4>(p.gamma + c0);
            const float* base = p.raw + ((size_t)it.b * s.L) * 3 * C + c0;
            Chunk a, b;
            // chunk k covers rows [whi - (k + 1) CH, whi - k CH)
            int t0 = whi - CH;
            chunk_load<true>(a, base, C, t0, wlo, whi);
            while (t0 + CH > wlo) {
                chunk_load<true>(b, base, C, t0 - CH, wlo, whi);
                chunk_fold(a, m, lr, li, gm, t0, wlo, whi);
                t0 -= CH;
                if (t0 + CH <= wlo) break;
                chunk_load<true>(a, base, C, t0 - CH, wlo, whi);
                chunk_fold(b, m, lr, li, gm, t0, wlo, whi);
                t0 -= CH;
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
    }

    // ---- scan: one counter per chain, every block composes its own prefix ----
    // Run maps sit on the rank's board as plain float4 per channel. A chain's counter counts
    // the runs that have arrived; the last one in sets it back to zero and writes the call's
    // epoch into the chain's ready word, so nothing is cleared between launches.
    FL_HD static float* runmap_at(const Params& p, size_t item, int ch) {
        return p.runmap + (item * kGroup + ch) * 4;
    }

    // end of sweep 1, channel threads: the run's map = the warps' maps in time order; it becomes
    // visible to the chain's other blocks
    FL_HD static void publish_run(const Params& p, int item, const Item& it, int thread, float* smem) {
        if (thread >= kGroup) return;
        Affine m = affine_identity();
        if (it.cg * kGroup + thread < p.s.C) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w)
                m = affine_then(m, sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]);
        }
        float* q = runmap_at(p, (size_t)item, thread);
#if FL_DEVICE_CODE
        __stcg(reinterpret_cast<float4*>(q), make_float4(m.ar, m.ai, m.br, m.bi));
#else
        q[0] = m.ar; q[1] = m.ai; q[2] = m.br; q[3] = m.bi;
#endif
    }
    // Runs after the block barrier that follows publish_run: the barrier orders the block's
    // stores before thread 0's arrival, which is a release (and acquire) at GPU scope, so
    // whoever sees the chain complete also sees every run's map.
    FL_HD static void arrive(const Params& p, const Item& it, int thread) {
        if (thread != 0) return;
        unsigned* word = p.count + it.chain;
#if FL_DEVICE_CODE
        unsigned old;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(word) : "memory");
        if (old == (unsigned)p.s.R - 1u) {
            // the last run in: the counter goes back to zero for the next launch (nobody else
            // touches it now) and the chain's ready word - a word of its own, so that the
            // blocks polling it stay off the counter's line - takes the epoch
            *word = 0u;
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ready + 64 * it.chain), "r"(p.epoch)
                         : "memory");
        }
#else
        if (++*word == (unsigned)p.s.R) {
            *word = 0u;
            p.ready[64 * it.chain] = p.epoch;
        }
#endif
    }

    FL_HD static unsigned* wait_flag(float* smem) {
        return reinterpret_cast<unsigned*>(smem + kSumFloats + kCarryFloats);
    }
    // thread 0: bounded wait until every run of the chain has arrived in this call
    FL_HD static void wait_chain(const Params& p, const Item& it, int thread, float* smem) {
        if (thread != 0) return;
        const unsigned want = p.epoch;
        const unsigned* word = p.ready + 64 * it.chain;
#if FL_DEVICE_CODE
        unsigned v, polls = 0;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
        while (v != want && ++polls < p.max_polls) {
            __nanosleep(polls < 64 ? 64 : 256);
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
        }
        wait_flag(smem)[0] = v == want ? 1u : 0u;
#else
        wait_flag(smem)[0] = *word == want ? 1u : 0u;
#endif
    }

    // Map from the span's start to the start of this run = the maps of the chain's earlier
    // runs in order. kThreads / 128 threads share a channel, each composes a contiguous share
    // of those runs, eight independent loads in flight; channel threads join the shares.
    static constexpr int kShares = kThreads / kGroup;
    static constexpr int kWindow = 8;
    FL_HD static float* share_at(float* smem, int h, int ch) {
        return smem + kSumFloats + ((size_t)h * kGroup + ch) * 4;   // the carry area, free here
    }
    FL_HD static float* prefix_at(float* smem, int k) {
        return smem + kSumFloats + kShares * kGroup * 4 + k * kGroup;
    }
    static_assert((kShares + 1) * kGroup * 4 <= kCarryFloats, "shares and prefix fit the carry area");

    FL_HD static Pub4 map_load(const float* q) {
#if FL_DEVICE_CODE
        const float4 t = __ldcg(reinterpret_cast<const float4*>(q));   // another block's store: L2
        return Pub4{t.x, t.y, t.z, t.w};
#else
        return Pub4{q[0], q[1], q[2], q[3]};
#endif
    }

    FL_HD static void prefix_shares(const Params& p, const Item& it, int thread, float* smem) {
        const int ch = thread % kGroup, h = thread / kGroup;
        if (h >= kShares) return;
        const int n = it.run;  // runs before this one
        const int per = (n + kShares - 1) / kShares;
        const int lo = h * per < n ? h * per : n;
        const int hi = lo + per < n ? lo + per : n;
        Affine m = affine_identity();
        if (wait_flag(smem)[0] == 0u) {  // the chain never completed: NaN from here on
            m.ar = m.ai = m.br = m.bi = nanf("");
#if FL_DEVICE_CODE
            atomicExch(p.error, 1u);
#else
            *p.error = 1u;
#endif
        } else if (it.cg * kGroup + ch < p.s.C) {
            const float* base = runmap_at(p, (size_t)it.chain, ch);
            const size_t stride = (size_t)p.s.chains * kGroup * 4;
            int j = lo;
            for (; j + kWindow <= hi; j += kWindow) {
                Pub4 v[kWindow];
#pragma unroll
                for (int u = 0; u < kWindow; ++u) v[u] = map_load(base + (size_t)(j + u) * stride);
#pragma unroll
                for (int u = 0; u < kWindow; ++u) m = affine_then(m, v[u].x, v[u].y, v[u].z, v[u].w);
            }
            for (; j < hi; ++j) {
                const Pub4 v = map_load(base + (size_t)j * stride);
                m = affine_then(m, v.x, v.y, v.z, v.w);
            }
        }
        float* o = share_at(smem, h, ch);
        o[0] = m.ar; o[1] = m.ai; o[2] = m.br; o[3] = m.bi;
    }

    // channel threads: join the shares; the owner of the chain's last run appends its own map,
    // which gives the span's map, and sends it to every rank
    FL_HD static void prefix_join(const Params& p, int item, const Item& it, int thread, float* smem) {
        const SpanShape& s = p.s;
        const int c = it.cg * kGroup + thread;
        if (thread >= kGroup || c >= s.C) return;
        Affine m = affine_identity();
#pragma unroll
        for (int h = 0; h < kShares; ++h) {
            const float* q = share_at(smem, h, thread);
            m = affine_then(m, q[0], q[1], q[2], q[3]);
        }
        if (it.run == s.R - 1) {
            const Pub4 own = map_load(runmap_at(p, (size_t)item, thread));
            const Affine t = affine_then(m, own.x, own.y, own.z, own.w);
            if (p.summary) {
                float* o = p.summary + (size_t)it.b * 4 * s.C + c;
                o[0] = t.ar; o[s.C] = t.ai; o[2 * (size_t)s.C] = t.br; o[3 * (size_t)s.C] = t.bi;
            }
            if (p.P > 1) {
                const size_t slot =
                    (((size_t)(p.epoch & 1u) * p.P + p.rank) * s.B + it.b) * 4 * s.C + c;
                // (a fixed trip count keeps the pointer table in the kernel's parameter space)
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r < p.P) {
                        MailPair* q = p.mailbox[r] + slot;
                        mail_store(q, t.ar, p.epoch);
                        mail_store(q + s.C, t.ai, p.epoch);
                        mail_store(q + 2 * (size_t)s.C, t.br, p.epoch);
                        mail_store(q + 3 * (size_t)s.C, t.bi, p.epoch);
                    }
                }
            }
        }
        prefix_at(smem, 0)[thread] = m.ar;
        prefix_at(smem, 1)[thread] = m.ai;
        prefix_at(smem, 2)[thread] = m.br;
        prefix_at(smem, 3)[thread] = m.bi;
    }

    // channel threads: state entering the run = prefix map of (earlier ranks folded onto
    // state0); from it, through the warps' maps of sweep 1, the state entering each warp's steps
    FL_HD static void enter_run(const Params& p, const Item& it, int thread, float* smem) {
        const SpanShape& s = p.s;
        const int c = it.cg * kGroup + thread;
        if (thread >= kGroup || c >= s.C) return;
        float sr = p.state0 ? p.state0[(size_t)it.b * 2 * s.C + c] : 0.0f;
        float si = p.state0 ? p.state0[(size_t)it.b * 2 * s.C + s.C + c] : 0.0f;
        bool failed = false;
        if (p.P > 1) {
            // two ranks' slots are fetched together (one L2 round trip for 8 pairs); a slot
            // found empty is then polled on its own, with the caller's bound
            for (int r0 = 0; r0 < p.P; r0 += kSpanMailWindow) {
                MailPair got[kSpanMailWindow][4];
#pragma unroll
                for (int w = 0; w < kSpanMailWindow; ++w) {
                    if (r0 + w < p.P) {
                        const MailPair* q = p.own +
                            (((size_t)(p.epoch & 1u) * p.P + r0 + w) * s.B + it.b) * 4 * s.C + c;
#pragma unroll
                        for (int k = 0; k < 4; ++k) got[w][k] = mail_load(q + (size_t)k * s.C);
                    }
                }
#pragma unroll
                for (int w = 0; w < kSpanMailWindow; ++w) {
                    if (r0 + w < p.P) {
                        const int r = r0 + w;
                        const MailPair* q = p.own +
                            (((size_t)(p.epoch & 1u) * p.P + r) * s.B + it.b) * 4 * s.C + c;
                        float v[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            MailPair m = got[w][k];
#if FL_DEVICE_CODE
                            unsigned polls = 0;
                            // a summary that is late ends the waiting for all that follow it
                            while (m.tag != p.epoch && !failed && ++polls < p.max_polls) {
                                backoff(polls);
                                m = mail_load(q + (size_t)k * s.C);
                            }
#endif
                            if (m.tag != p.epoch) failed = true;
                            v[k] = m.value;
                        }
                        if (!failed && r < p.rank) affine_apply(Affine{v[0], v[1], v[2], v[3]}, sr, si);
                    }
                }
            }
        }
        // (this thread's prefix entries share their place with carries it writes below: read first)
        const Affine pre{prefix_at(smem, 0)[thread], prefix_at(smem, 1)[thread],
                         prefix_at(smem, 2)[thread], prefix_at(smem, 3)[thread]};
        if (failed) {
#if FL_DEVICE_CODE
            atomicExch(p.error, 1u);
#else
            *p.error = 1u;
#endif
            sr = si = nanf("");
        } else {
            affine_apply(pre, sr, si);
        }
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            carry_at(smem, w, 0)[thread] = sr;
            carry_at(smem, w, 1)[thread] = si;
            affine_apply(Affine{sum_at(smem, w, 0)[thread], sum_at(smem, w, 1)[thread],
                                sum_at(smem, w, 2)[thread], sum_at(smem, w, 3)[thread]},
                         sr, si);
        }
        if (p.state_out && it.run == s.R - 1) {
            p.state_out[(size_t)it.b * 2 * s.C + c] = sr;
            p.state_out[(size_t)it.b * 2 * s.C + s.C + c] = si;
        }
    }

    // sweep 2, one chunk: gates, recurrence and displaced readout of its rows in time order,
    // streaming stores (reference :599-622)
    FL_HD static void chunk_emit(const Chunk& c, Vec<4>& sr, Vec<4>& si, const Vec<4>& lr,
                                 const Vec<4>& li, const Vec<4>& gm, float* obase, int C, int t0,
                                 int wlo, int whi) {
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const int t = t0 + u;
            if (t >= wlo && t < whi) {
                Vec<4> dr, di;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const Gate g = make_gate(c.zr[u].v[k], c.zi[u].v[k], c.zv[u].v[k]);
                    float mr, mi;
                    cmul(lr.v[k], li.v[k], sr.v[k], si.v[k], mr, mi);
                    dr.v[k] = g.vac * mr;
                    di.v[k] = g.vac * mi;
                    const float bs = gm.v[k] * g.vac;
                    sr.v[k] = (1.0f - g.vac) * mr + bs * g.inj_r;
                    si.v[k] = (1.0f - g.vac) * mi + bs * g.inj_i;
                }
                float* orow = obase + (size_t)t * 4 * C;
                vec_store_stream<4>(orow, sr);
                vec_store_stream<4>(orow + C, si);
                vec_store_stream<4>(orow + 2 * C, dr);
                vec_store_stream<4>(orow + 3 * C, di);
            }
        }
    }

    // Sweep 2 of one warp: its steps first to last from its entering state, two chunks in
    // flight, no block barrier anywhere.
    FL_HD static void sweep2_warp(const Params& p, const Item& it, int thread, float* smem) {
        const SpanShape& s = p.s;
        const int lane = thread & 31, warp = thread >> 5;
        const int C = s.C;
        const int c0 = it.cg * kGroup + lane * 4;
        int wlo, whi;
        warp_steps(it, warp, wlo, whi);
        if (c0 >= C || wlo >= whi) return;
        const Vec<4> lr = vec_load<4>(p.tr + c0);
        const Vec<4> li = vec_load<4>(p.ti + c0);
        const Vec<4> gm = vec_load<4>(p.gamma + c0);
        Vec<4> sr = vec_load<4>(carry_at(smem, warp, 0) + lane * 4);
        Vec<4> si = vec_load<4>(carry_at(smem, warp, 1) + lane * 4);
        const float* base = p.raw + ((size_t)it.b * s.L) * 3 * C + c0;
        float* obase = p.read + ((size_t)it.b * s.L) * 4 * C + c0;
        Chunk a, b;
        int t0 = wlo;
        chunk_load<false>(a, base, C, t0, wlo, whi);
        while (t0 < whi) {
            chunk_load<false>(b, base, C, t0 + CH, wlo, whi);
            chunk_emit(a, sr, si, lr, li, gm, obase, C, t0, wlo, whi);
            t0 += CH;
            if (t0 >= whi) break;
            chunk_load<false>(a, base, C, t0 + CH, wlo, whi);
            chunk_emit(b, sr, si, lr, li, gm, obase, C, t0, wlo, whi);
            t0 += CH;
        }
    }

    // The whole block program. `ex.all(f)` runs f(thread, state) for every thread of the block
    // and then synchronises the block (device: the calling thread, then __syncthreads(); host
    // emulation: a loop over the threads); `ex.run(f)` does the same without the barrier.
    // `ex.blocks()` is the grid size.
    template <class Exec>
    FL_HD static void run_block(const Params& p, int block, float* smem, Exec& ex) {
        const SpanShape& s = p.s;
        // A block with one item keeps its warps' maps in shared memory from sweep 1 to sweep 2;
        // otherwise (more items than blocks; the host emulation, which runs the parts apart)
        // the second part composes them again, from L2.
        const bool keeps_maps = s.items <= ex.blocks() && p.stages == 3;
        if (p.stages & 1) {
            for (int item = block; item < s.items; item += ex.blocks()) {
                const Item it = decode(s, item);
                ex.all([&](int t, State&) { sweep1_warp(p, it, t, smem); });
                ex.all([&](int t, State&) { publish_run(p, item, it, t, smem); });
                ex.run([&](int t, State&) { arrive(p, it, t); });
            }
        }
        if (p.stages & 6) {
            for (int item = block; item < s.items; item += ex.blocks()) {
                if (p.emu_round >= 0 && item != block + p.emu_round * ex.blocks()) continue;
                const Item it = decode(s, item);
                if (!keeps_maps && (p.stages & 2)) ex.run([&](int t, State&) { sweep1_warp(p, it, t, smem); });
                ex.all([&](int t, State&) { wait_chain(p, it, t, smem); });
                ex.all([&](int t, State&) { prefix_shares(p, it, t, smem); });
                ex.all([&](int t, State&) { prefix_join(p, item, it, t, smem); });
                if (!(p.stages & 2)) continue;  // host emulation: every rank sends before any waits
                ex.all([&](int t, State&) { enter_run(p, it, t, smem); });
                ex.all([&](int t, State&) { sweep2_warp(p, it, t, smem); });
            }
        }
    }
};

}  // namespace fields
