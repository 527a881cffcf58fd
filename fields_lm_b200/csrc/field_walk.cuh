// Chain-walking Field kernels for shapes with many independent chains (training).
//
// A chain is one batch row x 32 consecutive channels. One block owns one chain and
// walks it through time, tile by tile, with the state carried on chip, so blocks never
// wait for one another: no flags, no fences, no second read of anything. Tiles of the
// chain stream into shared memory through a ring of asynchronous 16-byte copies
// (cp.async) issued STAGES-1 tiles ahead, which keeps HBM requests in flight while
// the warps compute.
//
// Inside a tile, warp w owns TS consecutive steps and lane l owns channel l
// (shared-memory rows are 32 consecutive floats: conflict-free). Per tile:
//   A. each thread pulls its TS steps from shared memory into registers, evaluates the
//      gates once and composes the warp's affine map            -> maps[w]
//   B. each warp folds the maps of the warps before it onto the chain's running state,
//      then runs the recurrence over its registers and writes its outputs; the last warp
//      leaves the running state for the next tile.
// Two block barriers per tile. The same scheme runs backward in time for the gradient.
//
// Reference arithmetic: gates :493-501, recurrence and displaced readout :599-622,
// dual recurrence and gate derivatives :794-909 of
// field_only_v4_chunked_triton_wiki100.py.
#pragma once

#include "field_kernels.cuh"
#include "field_sync.cuh"

namespace fields {

constexpr int kLane = 32;  // channels per chain

struct WalkShape {
    int B, L, C;
    int NT;  // tiles per chain
    int G;   // 32-channel groups per row
};

struct WalkFwdParams {
    const float* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;  // [B, 2C] or null
    float* read;
    float* state_out;       // [B, 2C] or null
    WalkShape s;
};

template <int TS, int WARPS, int STAGES>
struct FwdWalk {
    using Params = WalkFwdParams;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = 1;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kStageFloats = kTile * 3 * kLane;
    static constexpr int kMapsOff = STAGES * kStageFloats;   // maps[WARPS][4][32]
    static constexpr int kRunOff = kMapsOff + WARPS * 4 * kLane;  // run[2][2][32]
    static constexpr int kSmemFloats = kRunOff + 2 * 2 * kLane;
    static constexpr int kChunksPerStep = 3 * (kLane / 4);  // 16-byte chunks per time step

    static constexpr int kCopies = kTile * kChunksPerStep / kThreads;  // copies per thread and tile
    static_assert(kTile * kChunksPerStep % kThreads == 0, "copies must divide evenly over threads");

    struct State {
        float br[TS], bi[TS], vac[TS];
        // this thread's copies of a tile, fixed for the whole walk: time row inside the tile
        // (or a huge value if the channel part lies past C), offsets in shared and global memory
        int crow[kCopies], csm[kCopies], cgl[kCopies];
    };

    FL_HD static int phases(const Params& p) { return 2 * p.s.NT + 1; }

    FL_HD static void plan_copies(const Params& p, int cg, int thread, State& st) {
        const WalkShape& s = p.s;
#pragma unroll
        for (int i = 0; i < kCopies; ++i) {
            const int q = thread + i * kThreads;
            const int t = q / kChunksPerStep;
            const int r = q % kChunksPerStep;
            const int plane = r / (kLane / 4);
            const int part = r % (kLane / 4);
            st.crow[i] = cg * kLane + part * 4 < s.C ? t : (1 << 30);
            st.csm[i] = (t * 3 + plane) * kLane + part * 4;
            st.cgl[i] = t * 3 * s.C + plane * s.C + part * 4;
        }
    }

    // Issues the copies of one tile into its ring slot (nothing for tiles past the end).
    FL_HD static void issue_tile(const Params& p, int b, int cg, int tile, float* smem,
                                 const State& st) {
        const WalkShape& s = p.s;
        if (tile < s.NT) {
            float* stage = smem + (tile % STAGES) * kStageFloats;
            const int t0 = tile * kTile;
            const float* base = p.raw + ((size_t)b * s.L + t0) * 3 * s.C + cg * kLane;
            const int rows = s.L - t0;  // rows of this tile that exist
#pragma unroll
            for (int i = 0; i < kCopies; ++i)
                if (st.crow[i] < rows) async_copy16(stage + st.csm[i], base + st.cgl[i]);
        }
        async_commit();
    }

    FL_HD static void phase(int ph, const Params& p, int block, int thread, float* smem, State& st) {
        const WalkShape& s = p.s;
        const int b = block / s.G, cg = block % s.G;
        const int lane = thread & 31, warp = thread >> 5;
        const int ch = cg * kLane + lane;
        const bool chan_ok = ch < s.C;
        float* maps = smem + kMapsOff;
        float* run = smem + kRunOff;

        if (ph == 0) {
            plan_copies(p, cg, thread, st);
            for (int j = 0; j < STAGES - 1; ++j) issue_tile(p, b, cg, j, smem, st);
            if (warp == 0) {
                run[lane] = (p.state_in && chan_ok) ? p.state_in[(size_t)b * 2 * s.C + ch] : 0.0f;
                run[kLane + lane] =
                    (p.state_in && chan_ok) ? p.state_in[(size_t)b * 2 * s.C + s.C + ch] : 0.0f;
            }
            async_wait_pending<STAGES - 2>();
            return;
        }
        const int tile = (ph - 1) >> 1;
        const int tw = tile * kTile + warp * TS;
        if ((ph - 1) & 1) {
            // B: fold the earlier warps' maps onto the running state, then the recurrence
            float* cur = run + (tile & 1) * 2 * kLane;
            float* nxt = run + ((tile + 1) & 1) * 2 * kLane;
            float sr = cur[lane], si = cur[kLane + lane];
            for (int w = 0; w < warp; ++w) {
                const float* m = maps + w * 4 * kLane + lane;
                affine_apply(Affine{m[0], m[kLane], m[2 * kLane], m[3 * kLane]}, sr, si);
            }
            if (chan_ok) {
                const float lr = p.tr[ch], li = p.ti[ch];
                float* obase = p.read + ((size_t)b * s.L + tw) * 4 * s.C + ch;
#pragma unroll
                for (int u = 0; u < TS; ++u) {
                    if (tw + u < s.L) {
                        float mr, mi;
                        cmul(lr, li, sr, si, mr, mi);
                        const float v = st.vac[u];
                        const float dr = v * mr, di = v * mi;
                        sr = (1.0f - v) * mr + st.br[u];
                        si = (1.0f - v) * mi + st.bi[u];
                        float* o = obase + u * 4 * s.C;
#if FL_DEVICE_CODE
                        __stcs(o, sr); __stcs(o + s.C, si);
                        __stcs(o + 2 * s.C, dr); __stcs(o + 3 * s.C, di);
#else
                        o[0] = sr; o[s.C] = si; o[2 * s.C] = dr; o[3 * s.C] = di;
#endif
                    }
                }
            }
            if (warp == WARPS - 1) {
                nxt[lane] = sr;
                nxt[kLane + lane] = si;
                if (tile == s.NT - 1 && p.state_out && chan_ok) {
                    p.state_out[(size_t)b * 2 * s.C + ch] = sr;
                    p.state_out[(size_t)b * 2 * s.C + s.C + ch] = si;
                }
            }
            async_wait_pending<STAGES - 2>();  // the next tile has landed (this thread's part)
        } else {
            // A: keep the ring full, then registers <- shared memory, gates, warp map
            issue_tile(p, b, cg, tile + STAGES - 1, smem, st);
            const float* stage = smem + (tile % STAGES) * kStageFloats;
            Affine m = affine_identity();
            if (chan_ok) {
                const float lr = p.tr[ch], li = p.ti[ch], gm = p.gamma[ch];
#pragma unroll
                for (int u = 0; u < TS; ++u) {
                    if (tw + u < s.L) {
                        const float* row = stage + ((warp * TS + u) * 3) * kLane + lane;
                        const Gate g = make_gate(row[0], row[kLane], row[2 * kLane]);
                        const float keep = 1.0f - g.vac;
                        const float bs = gm * g.vac;
                        st.br[u] = bs * g.inj_r;
                        st.bi[u] = bs * g.inj_i;
                        st.vac[u] = g.vac;
                        m = affine_then(m, keep * lr, keep * li, st.br[u], st.bi[u]);
                    }
                }
            }
            float* o = maps + warp * 4 * kLane + lane;
            o[0] = m.ar; o[kLane] = m.ai; o[2 * kLane] = m.br; o[3 * kLane] = m.bi;
        }
    }
};


// ---------------------------------------------------------------------------
// Backward chain walk: same structure, time runs from the last step to the first.
// A ring slot holds nine rows per step: z_r z_i z_v | u_r u_i gd_r gd_i | s_{t-1}
// (the last two from the saved forward output, row t-1). Tiles are visited from the
// end of the sequence; inside a tile warp 0 owns the latest steps.
// ---------------------------------------------------------------------------
struct WalkBwdParams {
    const float* raw;
    const float* tr;
    const float* ti;
    const float* gamma;
    const float* state_in;        // [B, 2C] or null
    const float* read;            // saved forward output
    const float* grad_read;
    const float* grad_state_out;  // [B, 2C] or null
    float* grad_raw;
    float* grad_state_in;         // [B, 2C] or null
    float* partial;               // [3][B][C]: one row of parameter-gradient sums per chain
    WalkShape s;
};

template <int TS, int WARPS, int STAGES>
struct BwdWalk {
    using Params = WalkBwdParams;
    static constexpr int kThreads = 32 * WARPS;
    static constexpr int kMinBlocks = 1;
    static constexpr int kTile = TS * WARPS;
    static constexpr int kRows = 9;
    static constexpr int kStageFloats = kTile * kRows * kLane;
    static constexpr int kMapsOff = STAGES * kStageFloats;        // maps[WARPS][4][32]
    static constexpr int kRunOff = kMapsOff + WARPS * 4 * kLane;  // run[2][2][32]
    static constexpr int kSmemFloats = kRunOff + 2 * 2 * kLane;
    static constexpr int kChunksPerStep = kRows * (kLane / 4);

    static constexpr int kCopies = kTile * kChunksPerStep / kThreads;
    static_assert(kTile * kChunksPerStep % kThreads == 0, "copies must divide evenly over threads");

    struct State {
        float inj_r[TS], inj_i[TS], sig[TS];  // gates
        float ur[TS], ui[TS], gdr[TS], gdi[TS], pr[TS], pi[TS];
        float dtr, dti, dgm;                   // running parameter-gradient sums of this thread
        // this thread's copies of a tile: time row inside the tile (huge if the channel part lies
        // past C), source (0 raw, 1 grad_read, 2 forward output one step earlier), offsets
        int crow[kCopies], ckind[kCopies], csm[kCopies], cgl[kCopies];
    };

    FL_HD static int phases(const Params& p) { return 2 * p.s.NT + 2; }

    FL_HD static void plan_copies(const Params& p, int cg, int thread, State& st) {
        const WalkShape& s = p.s;
#pragma unroll
        for (int i = 0; i < kCopies; ++i) {
            const int q = thread + i * kThreads;
            const int t = q / kChunksPerStep;
            const int r = q % kChunksPerStep;
            const int row = r / (kLane / 4);
            const int part = r % (kLane / 4);
            st.crow[i] = cg * kLane + part * 4 < s.C ? t : (1 << 30);
            st.csm[i] = (t * kRows + row) * kLane + part * 4;
            st.ckind[i] = row < 3 ? 0 : (row < 7 ? 1 : 2);
            st.cgl[i] = row < 3 ? t * 3 * s.C + row * s.C + part * 4
                                : t * 4 * s.C + (row < 7 ? row - 3 : row - 7) * s.C + part * 4;
        }
    }

    // Scan-order tile j covers time tile NT-1-j.
    FL_HD static void issue_tile(const Params& p, int b, int cg, int j, float* smem,
                                 const State& st) {
        const WalkShape& s = p.s;
        if (j < s.NT) {
            float* stage = smem + (j % STAGES) * kStageFloats;
            const long long t0 = (long long)(s.NT - 1 - j) * kTile;
            const long long row0 = (long long)b * s.L + t0;
            const float* zb = p.raw + row0 * 3 * s.C + cg * kLane;
            const float* gb = p.grad_read + row0 * 4 * s.C + cg * kLane;
            // one step earlier; for t0 = 0 the first row is never read (s_{-1} is the incoming state)
            const float* rb = p.read + (row0 - 1) * 4 * s.C + cg * kLane;
            const int rows = s.L - (int)t0;
            const int first_prev = t0 == 0 ? 1 : 0;
#pragma unroll
            for (int i = 0; i < kCopies; ++i) {
                if (st.crow[i] >= rows) continue;
                if (st.ckind[i] == 0) {
                    async_copy16(stage + st.csm[i], zb + st.cgl[i]);
                } else if (st.ckind[i] == 1) {
                    async_copy16(stage + st.csm[i], gb + st.cgl[i]);
                } else if (st.crow[i] >= first_prev) {
                    async_copy16(stage + st.csm[i], rb + st.cgl[i]);
                }
            }
        }
        async_commit();
    }

    FL_HD static void phase(int ph, const Params& p, int block, int thread, float* smem, State& st) {
        const WalkShape& s = p.s;
        const int b = block / s.G, cg = block % s.G;
        const int lane = thread & 31, warp = thread >> 5;
        const int ch = cg * kLane + lane;
        const bool chan_ok = ch < s.C;
        float* maps = smem + kMapsOff;
        float* run = smem + kRunOff;

        if (ph == 0) {
            plan_copies(p, cg, thread, st);
            for (int j = 0; j < STAGES - 1; ++j) issue_tile(p, b, cg, j, smem, st);
            if (warp == 0) {
                const bool have = p.grad_state_out && chan_ok;
                run[lane] = have ? p.grad_state_out[(size_t)b * 2 * s.C + ch] : 0.0f;
                run[kLane + lane] = have ? p.grad_state_out[(size_t)b * 2 * s.C + s.C + ch] : 0.0f;
            }
            st.dtr = st.dti = st.dgm = 0.0f;
            async_wait_pending<STAGES - 2>();
            return;
        }
        if (ph == 2 * s.NT + 1) {
            // every warp has left its sums at the start of the (now idle) ring; add them in a
            // fixed order
            if (warp == 0 && chan_ok) {
                const size_t plane = (size_t)s.B * s.C;
                float* out = p.partial + (size_t)b * s.C + ch;
                for (int k = 0; k < 3; ++k) {
                    float acc = 0.0f;
                    for (int w = 0; w < WARPS; ++w) acc += smem[(w * 3 + k) * kLane + lane];
                    out[k * plane] = acc;
                }
            }
            return;
        }
        const int j = (ph - 1) >> 1;                      // tile in scan order
        const int tile_lo = (s.NT - 1 - j) * kTile;       // first time step of the tile
        const int tbeg = tile_lo + (WARPS - 1 - warp) * TS;  // warp 0 owns the latest steps
        const int slot_row = (WARPS - 1 - warp) * TS;     // row of tbeg inside the ring slot

        if ((ph - 1) & 1) {
            // B: carry from the later-in-time warps, then the reverse recurrence
            float* cur = run + (j & 1) * 2 * kLane;
            float* nxt = run + ((j + 1) & 1) * 2 * kLane;
            float cr = cur[lane], ci = cur[kLane + lane];
            for (int w = 0; w < warp; ++w) {
                const float* m = maps + w * 4 * kLane + lane;
                affine_apply(Affine{m[0], m[kLane], m[2 * kLane], m[3 * kLane]}, cr, ci);
            }
            if (chan_ok) {
                const float lr = p.tr[ch], li = p.ti[ch], gm = p.gamma[ch];
                float* obase = p.grad_raw + ((size_t)b * s.L + tbeg) * 3 * s.C + ch;
#pragma unroll
                for (int uu = 0; uu < TS; ++uu) {
                    const int u = TS - 1 - uu;  // descending in time
                    const int t = tbeg + u;
                    if (t < s.L) {
                        const float vac = kVacMax * st.sig[u];
                        const float keep = 1.0f - vac;
                        const float Gr = st.ur[u] + cr, Gi = st.ui[u] + ci;
                        const float gdr = st.gdr[u], gdi = st.gdi[u];
                        const float sr = st.pr[u], si = st.pi[u];
                        float mr, mi, dar, dai, xr, xi, yr, yi, nr, ni;
                        cmul(lr, li, sr, si, mr, mi);
                        cmul_conj(sr, si, Gr, Gi, dar, dai);
                        cmul_conj(sr, si, gdr, gdi, xr, xi);
                        cmul_conj(lr, li, gdr, gdi, yr, yi);
                        cmul_conj(keep * lr, keep * li, Gr, Gi, nr, ni);
                        const float common_b = st.inj_r[u] * Gr + st.inj_i[u] * Gi;
                        const float dv = -lr * dar - li * dai + gm * common_b + gdr * mr + gdi * mi;
                        st.dtr += keep * dar + vac * xr;
                        st.dti += keep * dai + vac * xi;
                        st.dgm += vac * common_b;
                        const float bs = gm * vac;
                        const float ozr = bs * Gr * (1.0f - st.inj_r[u] * st.inj_r[u]);
                        const float ozi = bs * Gi * (1.0f - st.inj_i[u] * st.inj_i[u]);
                        const float ozv = dv * kVacMax * st.sig[u] * (1.0f - st.sig[u]);
                        float* o = obase + u * 3 * s.C;
#if FL_DEVICE_CODE
                        __stcs(o, ozr); __stcs(o + s.C, ozi); __stcs(o + 2 * s.C, ozv);
#else
                        o[0] = ozr; o[s.C] = ozi; o[2 * s.C] = ozv;
#endif
                        cr = nr + vac * yr;
                        ci = ni + vac * yi;
                    }
                }
            }
            if (warp == WARPS - 1) {
                nxt[lane] = cr;
                nxt[kLane + lane] = ci;
                if (j == s.NT - 1 && p.grad_state_in && chan_ok) {
                    p.grad_state_in[(size_t)b * 2 * s.C + ch] = cr;
                    p.grad_state_in[(size_t)b * 2 * s.C + s.C + ch] = ci;
                }
            }
            if (j == s.NT - 1) {
                // last tile: hand the thread's parameter-gradient sums to the final phase. Every
                // copy into the ring has landed and its data is in registers, so the ring is free;
                // the maps are still being read by slower warps.
                float* o = smem + warp * 3 * kLane + lane;
                o[0] = st.dtr; o[kLane] = st.dti; o[2 * kLane] = st.dgm;
            }
            async_wait_pending<STAGES - 2>();
        } else {
            // A: keep the ring full; registers <- shared memory; gates; warp's dual map
            issue_tile(p, b, cg, j + STAGES - 1, smem, st);
            const float* stage = smem + (j % STAGES) * kStageFloats;
            Affine m = affine_identity();
            if (chan_ok) {
                const float lr = p.tr[ch], li = p.ti[ch];
#pragma unroll
                for (int uu = 0; uu < TS; ++uu) {
                    const int u = TS - 1 - uu;
                    const int t = tbeg + u;
                    if (t < s.L) {
                        const float* row = stage + ((slot_row + u) * kRows) * kLane + lane;
                        const Gate g = make_gate(row[0], row[kLane], row[2 * kLane]);
                        st.inj_r[u] = g.inj_r; st.inj_i[u] = g.inj_i; st.sig[u] = g.sig;
                        st.ur[u] = row[3 * kLane]; st.ui[u] = row[4 * kLane];
                        st.gdr[u] = row[5 * kLane]; st.gdi[u] = row[6 * kLane];
                        if (t > 0) {
                            st.pr[u] = row[7 * kLane]; st.pi[u] = row[8 * kLane];
                        } else {
                            st.pr[u] = p.state_in ? p.state_in[(size_t)b * 2 * s.C + ch] : 0.0f;
                            st.pi[u] = p.state_in ? p.state_in[(size_t)b * 2 * s.C + s.C + ch] : 0.0f;
                        }
                        const float keep = 1.0f - g.vac;
                        const float car = keep * lr, cai = -keep * li;
                        float qr, qi, xr, xi;
                        cmul(car, cai, st.ur[u], st.ui[u], qr, qi);
                        cmul_conj(lr, li, st.gdr[u], st.gdi[u], xr, xi);
                        m = affine_then(m, car, cai, qr + g.vac * xr, qi + g.vac * xi);
                    }
                }
            }
            float* o = maps + warp * 4 * kLane + lane;
            o[0] = m.ar; o[kLane] = m.ai; o[2 * kLane] = m.br; o[3 * kLane] = m.bi;
        }
    }
};

}  // namespace fields
