// C ABI of the Field-recurrence library: argument checks, the launch plan and
// the kernel launches. Declarations and the contract of every entry point are
// in include/fields_read.h.
//
// Compiled by nvcc for sm_100a into libfields_read.so. The CPU tests compile
// this same file with g++ and FIELDS_HOST_EMU defined: launches then become
// nested loops over (block, phase, thread) on host memory, so the plan, the
// index arithmetic and the formulas are checked without a GPU. That build is
// test infrastructure; it is never loaded by the package.
#include "field_kernels.cuh"
#include "field_singlepass.cuh"
#ifdef FIELDS_ALL_VARIANTS
#include "field_walk.cuh"
#endif
#include "field_span.cuh"
#include "field_tensor.cuh"
#include "field_scan.cuh"
#include "field_epilogue.cuh"

#include "../../include/fields_read.h"

#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

namespace fields {

// ---------------------------------------------------------------------------
// Launch machinery
// ---------------------------------------------------------------------------
#ifdef FIELDS_HOST_EMU

using Stream = void*;
static thread_local const char* g_last_error = "no error";

template <class K>
static int launch(const typename K::Params& p, long long grid, Stream) {
    std::vector<double> smem_store((K::kSmemFloats + 1) / 2 + 1);  // double-aligned
    float* smem = reinterpret_cast<float*>(smem_store.data());
    for (long long block = 0; block < grid; ++block) {
        for (int thread = 0; thread < K::kThreads; ++thread) K::phase0(p, (int)block, thread, smem);
        if constexpr (K::kPhases > 1) {
            for (int thread = 0; thread < K::kThreads; ++thread)
                K::phase1(p, (int)block, thread, smem);
        }
    }
    return FIELDS_OK;
}

static int fill_zero(float* p, size_t n, Stream) {
    for (size_t i = 0; i < n; ++i) p[i] = 0.0f;
    return FIELDS_OK;
}

template <class K, int PH>
static void emu_phase_range(const typename K::Params& p, int block, float* smem,
                            typename K::State* st, int lo, int hi) {
    if constexpr (PH < K::kPhases) {
        if (PH >= lo && PH < hi)
            for (int thread = 0; thread < K::kThreads; ++thread)
                K::template phase<PH>(p, block, thread, smem, st[thread]);
        emu_phase_range<K, PH + 1>(p, block, smem, st, lo, hi);
    }
}

// Kernels whose blocks wait for one another: every block first runs up to the point
// where it has published its aggregate, then the blocks finish one at a time. With
// FIELDS_EMU_ORDER=reverse the later tiles finish first (after the first tile of each
// chain), which drives the look-back through whole chains of aggregates; the default
// order meets an inclusive state at the first step back.
template <class K>
static int launch_stateful(const typename K::Params& p, long long grid, long long first_wave,
                           Stream) {
    std::vector<double> smem_store((size_t)grid * (K::kSmemFloats / 2 + 1));
    std::vector<typename K::State> states((size_t)grid * K::kThreads);
    auto smem_of = [&](long long b) {
        return reinterpret_cast<float*>(smem_store.data() + (size_t)b * (K::kSmemFloats / 2 + 1));
    };
    for (long long b = 0; b < grid; ++b)
        emu_phase_range<K, 0>(p, (int)b, smem_of(b), &states[(size_t)b * K::kThreads], 0,
                              K::kSplitPhase);
    const char* order = std::getenv("FIELDS_EMU_ORDER");
    const bool reverse = order && std::string(order) == "reverse";
    std::vector<long long> seq;
    for (long long b = 0; b < first_wave && b < grid; ++b) seq.push_back(b);
    if (reverse) for (long long b = grid - 1; b >= first_wave; --b) seq.push_back(b);
    else for (long long b = first_wave; b < grid; ++b) seq.push_back(b);
    for (long long b : seq)
        emu_phase_range<K, 0>(p, (int)b, smem_of(b), &states[(size_t)b * K::kThreads],
                              K::kSplitPhase, K::kPhases);
    return FIELDS_OK;
}

static int fill_unset(void* p, size_t bytes, Stream) {
    std::memset(p, kUnsetByte, bytes);
    return FIELDS_OK;
}

// A staged kernel in the emulation: one tile per block, every tile stages its own rows.
template <class K>
static int launch_persistent(const typename K::Params& p, long long grid, long long first_wave,
                             Stream st) {
    return launch_stateful<K>(p, grid, first_wave, st);
}


template <class K>
static int resident_blocks() { return 4; }  // any positive distance exercises the prefetch path

// Persistent kernels written as one block program over an executor (field_span.cuh): the
// blocks run one after another, every phase as a loop over the block's threads.
template <class K>
struct EmuExec {
    typename K::State* states;
    int nblocks;
    template <class F> void all(F f) { for (int t = 0; t < K::kThreads; ++t) f(t, states[t]); }
    template <class F> void run(F f) { all(f); }
    int blocks() const { return nblocks; }
};

template <class K>
static int launch_span(const typename K::Params& p, int grid, Stream) {
    std::vector<double> smem_store(K::kSmemFloats / 2 + 1);
    float* smem = reinterpret_cast<float*>(smem_store.data());
    std::vector<typename K::State> states(K::kThreads);
    for (int block = 0; block < grid; ++block) {
        EmuExec<K> ex{states.data(), grid};
        typename K::Params q = p;
        q.stages = p.stages & 1;  // every block's first sweep (and the scans) before any wait
        K::run_block(q, block, smem, ex);
    }
    // second part item by item in index order (a block's later items may need maps that blocks
    // with a higher index produce in an earlier round; on the GPU those run concurrently)
    const int rounds = (p.s.items + grid - 1) / grid;
    for (int round = 0; round < rounds; ++round) {
        for (int block = 0; block < grid; ++block) {
            EmuExec<K> ex{states.data(), grid};
            typename K::Params q = p;
            q.stages = p.stages & 6;
            q.emu_round = round;
            K::run_block(q, block, smem, ex);
        }
    }
    return FIELDS_OK;
}

static int g_emu_span_stages = 3;

template <class K>
static int span_grid() { return 6; }  // a handful of blocks: several runs per chain, several items per block

// Kernels whose number of barrier-separated phases depends on the extents.
template <class K>
static int launch_walk(const typename K::Params& p, long long grid, Stream) {
    std::vector<double> smem_store(K::kSmemFloats / 2 + 1);
    float* smem = reinterpret_cast<float*>(smem_store.data());
    std::vector<typename K::State> states(K::kThreads);
    const int n = K::phases(p);
    for (long long block = 0; block < grid; ++block)
        for (int ph = 0; ph < n; ++ph)
            for (int thread = 0; thread < K::kThreads; ++thread)
                K::phase(ph, p, (int)block, thread, smem, states[thread]);
    return FIELDS_OK;
}

#else  // real CUDA build

using Stream = cudaStream_t;
static thread_local const char* g_last_error = "no error";

// Programmatic dependent launch. Every kernel of this library is launched with the
// programmatic-serialization attribute and begins by waiting, before it touches any memory,
// until the kernel before it on the stream has completed and its writes are visible. The
// launch itself (grid set-up, block scheduling) then overlaps the end of the previous kernel
// instead of following it. Because every kernel waits, the completion order of the stream is
// kept along the whole chain. No kernel signals early: letting the next grid take SM slots
// while this one still ran its last blocks was measured and was slower. The instruction does
// nothing in a kernel launched without the attribute (FIELDS_READ_PDL=0).
__device__ __forceinline__ void wait_for_previous_kernel() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

static bool dependent_launch_from_env() {
    const char* e = std::getenv("FIELDS_READ_PDL");
    return !(e && e[0] == '0');
}
#ifdef FIELDS_ALL_VARIANTS
static bool dependent_launch_enabled() { return dependent_launch_from_env(); }  // test build: per call
#else
// (the environment is read once, at the first launch)
static bool dependent_launch_enabled() {
    static const bool enabled = dependent_launch_from_env();
    return enabled;
}
#endif

template <class K>
__global__ void __launch_bounds__(K::kThreads) kernel_entry(const typename K::Params p) {
    extern __shared__ __align__(16) float smem[];
    wait_for_previous_kernel();
    K::phase0(p, (int)blockIdx.x, (int)threadIdx.x, smem);
    if constexpr (K::kPhases > 1) {
        __syncthreads();
        K::phase1(p, (int)blockIdx.x, (int)threadIdx.x, smem);
    }
}

static int check_cuda(cudaError_t e) {
    if (e == cudaSuccess) return FIELDS_OK;
    g_last_error = cudaGetErrorString(e);
    return FIELDS_ERR_LAUNCH;
}

// One launch, with the programmatic-serialization attribute unless FIELDS_READ_PDL=0.
template <class P>
static int launch_on(void (*fn)(const P), unsigned grid, unsigned threads, size_t bytes, Stream st,
                     const P& params) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, fn, params));
}

template <class K>
static int launch(const typename K::Params& p, long long grid, Stream st) {
    if (grid <= 0) return FIELDS_OK;
    if (grid > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    return launch_on<typename K::Params>(kernel_entry<K>, (unsigned)grid, K::kThreads,
                                         K::kSmemFloats * sizeof(float), st, p);
}

static int fill_zero(float* p, size_t n, Stream st) {
    return check_cuda(cudaMemsetAsync(p, 0, n * sizeof(float), st));
}

// Phases FIRST..LAST of one tile, with the block barriers between them.
template <class K, int PH, int LAST>
__device__ __forceinline__ void run_phases(const typename K::Params& p, int tile, float* smem,
                                           typename K::State& st) {
    K::template phase<PH>(p, tile, (int)threadIdx.x, smem, st);
    if constexpr (PH < LAST) {
        if constexpr (K::barrier_after(PH)) __syncthreads();
        run_phases<K, PH + 1, LAST>(p, tile, smem, st);
    }
}

// One block per tile, taken in block-index order (time-major): every tile a block may wait
// for has a smaller index, so the hardware has already started it. (A persistent variant
// that claimed tiles from a counter was measured and was no faster: the claim sits on the
// critical path and the loop costs registers.) After the look-back, while the last sweep
// runs, the block can warm L2 with the inputs of the tile `prefetch` positions ahead, which
// is about the tile that the block taking this one's place will read.
// The order in which tiles are handed out. By default the tile is the block index: a tile's
// predecessors then have smaller block indices, and the kernels rely on the hardware starting
// blocks in index order (what every CUDA GPU so far does, though the programming model does not
// promise it; if a GPU ever did otherwise a block could wait, up to its bound, for a block that
// has not started, and the call would end with FIELDS_ERR_TIMEOUT, not hang). With `s.ticket` set
// a block instead takes its tile from a counter in the workspace header (word 1, which the fill
// leaves at 0xFFFFFFFF, so the first ticket is 0): predecessors then belong to blocks that took
// their tickets earlier and are running, whatever the dispatch order. The atomic's round trip
// sits at the head of every tile: measured +9.5 % on the forward, +3.7 % on the fp32 step and
// +10 % on the bfloat16 step at 8 x 2,048 tokens, which is why it is off in the product and
// selectable (FIELDS_TILE_TICKET=1) only in the test build, where the GPU tests run it.
template <class K>
__global__ void __launch_bounds__(K::kThreads, K::kMinBlocks) stateful_entry(const typename K::Params p) {
    extern __shared__ __align__(16) float smem[];
    typename K::State st;
    wait_for_previous_kernel();
    int tile = (int)blockIdx.x;
#ifdef FIELDS_ALL_VARIANTS
    if (p.s.ticket) {
        // handed round through the first word of the carry area, which no phase writes before
        // the barrier that follows phase 0
        int* ticket = reinterpret_cast<int*>(smem + K::kSumFloats);
        if (threadIdx.x == 0) *ticket = (int)(atomicAdd(p.ctrl + 1, 1u) + 1u);
        __syncthreads();
        tile = *ticket;
    }
#endif
    run_phases<K, 0, K::kClaimAfter>(p, tile, smem, st);
    __syncthreads();
    if (p.s.prefetch > 0) {
        const long long next = (long long)tile + p.s.prefetch;
        if (next < (long long)p.s.B * p.s.G * p.s.NT) K::prefetch(p, (int)next, (int)threadIdx.x);
    }
    run_phases<K, K::kClaimAfter + 1, K::kPhases - 1>(p, tile, smem, st);
}

// Persistent form for kernels with staging cells (K::kStaged). Blocks take tiles from a ticket
// counter (word 1 of the workspace header, which the fill leaves at 0xFFFFFFFF, so the first
// ticket is 0), always one tile ahead: thread 0 issues the atomic for the next ticket at the top
// of a tile and hands its result round after phase 0, when every thread starts the copies of
// the next tile's rows into its staging cells.
template <class K>
__global__ void __launch_bounds__(K::kThreads, K::kMinBlocks) persistent_entry(const typename K::Params p) {
    extern __shared__ __align__(16) float smem[];
    typename K::State st;
    const unsigned tiles = (unsigned)((long long)p.s.B * p.s.G * p.s.NT);
    unsigned* hand = K::ticket_at(smem);
    wait_for_previous_kernel();
    if (threadIdx.x == 0) *hand = atomicAdd(p.ctrl + 1, 1u) + 1u;
    __syncthreads();
    unsigned tile = *hand;
    if (tile < tiles) K::stage(p, (int)tile, (int)threadIdx.x, smem);
    while (tile < tiles) {
        unsigned next_ticket = 0;
        if (threadIdx.x == 0) next_ticket = atomicAdd(p.ctrl + 1, 1u) + 1u;  // used after phase 0
        K::template phase<0>(p, (int)tile, (int)threadIdx.x, smem, st);
        if (threadIdx.x == 0) *hand = next_ticket;
        __syncthreads();
        const unsigned next = *hand;
        if (next < tiles) K::stage(p, (int)next, (int)threadIdx.x, smem);
        run_phases<K, 1, K::kPhases - 1>(p, (int)tile, smem, st);
        __syncthreads();  // the map, carry and hand-over areas are written again by the next tile
        tile = next;
    }
}

// Kernels that need more than the default 48 KB of dynamic shared memory opt in once per device.
// `ready` is the caller's per-kernel, per-device record (kernels of equal signature share a
// function-pointer type, so the record cannot live in this template).
template <class Fn>
static int allow_shared_memory(Fn fn, size_t bytes, bool* ready) {
    if (bytes <= 48 * 1024) return FIELDS_OK;
    static std::mutex mu;
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return FIELDS_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (!ready[dev]) {
        rc = check_cuda(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)bytes));
        if (rc) return rc;
        ready[dev] = true;
    }
    return FIELDS_OK;
}

// (the third argument, the number of chains, only matters to the host emulation)
template <class K>
static int launch_stateful(const typename K::Params& p, long long tiles, long long, Stream st) {
    if (tiles <= 0) return FIELDS_OK;
    if (tiles > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    constexpr size_t bytes = K::kSmemFloats * sizeof(float);
    static bool ready[64] = {};
    const int rc = allow_shared_memory(stateful_entry<K>, bytes, ready);
    if (rc) return rc;
    return launch_on<typename K::Params>(stateful_entry<K>, (unsigned)tiles, K::kThreads, bytes, st, p);
}

// Fills with the "not yet written" pattern. A kernel rather than a memset, so that it takes part
// in the dependent-launch chain: a memset would make the kernel after it wait for a full drain.
struct FillParams {
    uint4* p;
    size_t n;  // 16-byte words
};
constexpr int kFillThreads = 256, kFillPerThread = 4;

__global__ void __launch_bounds__(kFillThreads) fill_entry(const FillParams q) {
    wait_for_previous_kernel();
    const size_t base = (size_t)blockIdx.x * (kFillThreads * kFillPerThread) + threadIdx.x;
#pragma unroll
    for (int j = 0; j < kFillPerThread; ++j) {
        const size_t i = base + (size_t)j * kFillThreads;
        if (i < q.n) q.p[i] = make_uint4(kUnsetBits, kUnsetBits, kUnsetBits, kUnsetBits);
    }
}

static int fill_unset(void* p, size_t bytes, Stream st) {
    if (!dependent_launch_enabled() || (reinterpret_cast<uintptr_t>(p) & 15) || (bytes & 15))
        return check_cuda(cudaMemsetAsync(p, kUnsetByte, bytes, st));
    const size_t n = bytes / 16, per_block = (size_t)kFillThreads * kFillPerThread;
    if (n == 0) return FIELDS_OK;
    return launch_on<FillParams>(fill_entry, (unsigned)((n + per_block - 1) / per_block), kFillThreads,
                                 0, st, FillParams{static_cast<uint4*>(p), n});
}

// Blocks of kernel K that the current GPU holds at once (occupancy x SM count), asked once per device.
template <class K>
static int resident_blocks() {
    static std::mutex mu;
    static int cached[64] = {};
    int per_sm = 0, dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, stateful_entry<K>, K::kThreads,
                                                      K::kSmemFloats * sizeof(float)) != cudaSuccess)
        return 0;
    cached[dev] = per_sm * sms;
    return cached[dev];
}

// Launch of a staged kernel as persistent blocks: as many as the GPU holds at once (asked once
// per device, after the opt-in to its shared memory; fewer resident blocks only make it slower,
// the tickets keep it correct), never more than there are tiles.
template <class K>
static int launch_persistent(typename K::Params p, long long tiles, long long, Stream st) {
    if (tiles <= 0) return FIELDS_OK;
    if (tiles > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    constexpr size_t bytes = K::kSmemFloats * sizeof(float);
    static bool ready[64] = {};
    int rc = allow_shared_memory(persistent_entry<K>, bytes, ready);
    if (rc) return rc;
    static std::mutex mu;
    static int cached[64] = {};
    int dev = 0, resident = 0;
    rc = check_cuda(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return FIELDS_ERR_UNSUPPORTED;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (cached[dev] == 0) {
            int per_sm = 0, sms = 0;
            rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            if (!rc)
                rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                    &per_sm, persistent_entry<K>, K::kThreads, bytes));
            if (rc) return rc;
            if (per_sm * sms <= 0) return FIELDS_ERR_UNSUPPORTED;
            cached[dev] = per_sm * sms;
        }
        resident = cached[dev];
    }
    const long long grid = tiles < resident ? tiles : resident;
    return launch_on<typename K::Params>(persistent_entry<K>, (unsigned)grid, K::kThreads, bytes, st, p);
}

// Persistent block program over an executor: the calling thread, then a block barrier.
template <class K>
struct DeviceExec {
    typename K::State& st;
    template <class F> __device__ __forceinline__ void all(F f) { f((int)threadIdx.x, st); __syncthreads(); }
    template <class F> __device__ __forceinline__ void run(F f) { f((int)threadIdx.x, st); }
    __device__ __forceinline__ int blocks() const { return (int)gridDim.x; }
};

template <class K>
__global__ void __launch_bounds__(K::kThreads, K::kMinBlocks) span_entry(const typename K::Params p) {
    extern __shared__ __align__(16) float smem[];
    typename K::State st;
    DeviceExec<K> ex{st};
    wait_for_previous_kernel();
    if (p.epoch_word == nullptr) {
        K::run_block(p, (int)blockIdx.x, smem, ex);
        return;
    }
    // Epoch kept on the device: every block reads the last completed epoch when it starts; the
    // block that finishes last (all others have read it long before) stores the new one. The
    // ranks' counters advance together because every rank makes the same calls.
    typename K::Params q = p;
    unsigned last;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(last) : "l"(p.epoch_word) : "memory");
    q.epoch = last + 1u ? last + 1u : 1u;   // never 0
    K::run_block(q, (int)blockIdx.x, smem, ex);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.epoch_word + 1, 1u) == gridDim.x - 1) {
            p.epoch_word[1] = 0;
            __threadfence();
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.epoch_word), "r"(q.epoch) : "memory");
        }
    }
}

// Blocks of span_entry<K> that the current device holds at once, asked once per device.
template <class K>
static int span_grid() {
    static std::mutex mu;
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] <= 0) {
        int per_sm = 0, sms = 0;
        // (the opt-in to more than 48 KB of shared memory comes first: the query depends on it)
        if (K::kSmemFloats * sizeof(float) > 48 * 1024 &&
            cudaFuncSetAttribute(span_entry<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(K::kSmemFloats * sizeof(float))) != cudaSuccess)
            return 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, span_entry<K>, K::kThreads,
                                                          K::kSmemFloats * sizeof(float)) != cudaSuccess)
            return 0;
        cached[dev] = per_sm * sms;
    }
    return cached[dev];
}

// Cooperative launch (all blocks resident at once: they wait for one another), with the
// programmatic-serialization attribute beside it where the driver accepts the pair.
template <class K>
static int launch_span(const typename K::Params& p, int grid, Stream st) {
    if (grid <= 0) return FIELDS_ERR_LAUNCH;
    constexpr size_t bytes = K::kSmemFloats * sizeof(float);
    static bool ready[64] = {};
    int rc = allow_shared_memory(span_entry<K>, bytes, ready);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(K::kThreads);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static bool pair_refused = false;
    cfg.numAttrs = (dependent_launch_enabled() && !pair_refused) ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, span_entry<K>, p);
    if (e != cudaSuccess && cfg.numAttrs == 2) {
        (void)cudaGetLastError();
        pair_refused = true;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, span_entry<K>, p);
    }
    return check_cuda(e);
}

template <class K>
__global__ void __launch_bounds__(K::kThreads, K::kMinBlocks) walk_entry(const typename K::Params p) {
    extern __shared__ __align__(16) float smem[];
    typename K::State st;
    wait_for_previous_kernel();
    const int n = K::phases(p);
    for (int ph = 0; ph < n; ++ph) {
        K::phase(ph, p, (int)blockIdx.x, (int)threadIdx.x, smem, st);
        __syncthreads();
    }
}

template <class K>
static int launch_walk(const typename K::Params& p, long long grid, Stream st) {
    if (grid <= 0) return FIELDS_OK;
    if (grid > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    constexpr size_t bytes = K::kSmemFloats * sizeof(float);
    static bool ready[64] = {};
    const int rc = allow_shared_memory(walk_entry<K>, bytes, ready);
    if (rc) return rc;
    return launch_on<typename K::Params>(walk_entry<K>, (unsigned)grid, K::kThreads, bytes, st, p);
}

#endif

// ---------------------------------------------------------------------------
// Plan: chunk length and workspace layout, a function of the extents only.
// ---------------------------------------------------------------------------
constexpr long long kTargetWarps = 148LL * 32;  // enough warps to fill every SM of a B200

struct Plan {
    Shape s;             // with G for the vector width in use
    size_t plane;        // B * N * C floats
    size_t sum_off, carry_off, partial_off;  // in floats
    size_t fwd_floats, bwd_floats;
};

static size_t round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

static Plan make_plan(int B, int L, int C, int vec) {
    Plan pl{};
    const int nominal_vec = (C % 4 == 0) ? 4 : 1;
    const long long groups = (C + 32 * nominal_vec - 1) / (32 * nominal_vec);
    int ts = 16;
    const int candidates[3] = {64, 32, 16};
    for (int k = 0; k < 3; ++k) {
        const long long n = (L + candidates[k] - 1) / candidates[k];
        if ((long long)B * n * groups >= kTargetWarps) { ts = candidates[k]; break; }
    }
    pl.s.B = B; pl.s.L = L; pl.s.C = C;
    pl.s.ts = ts;
    pl.s.N = (L + ts - 1) / ts;
    pl.s.G = (C + 32 * vec - 1) / (32 * vec);
    pl.plane = (size_t)B * pl.s.N * C;
    pl.sum_off = 0;
    pl.carry_off = round_up(4 * pl.plane, 64);
    pl.partial_off = pl.carry_off + round_up(2 * pl.plane, 64);
    pl.fwd_floats = pl.partial_off;
    pl.bwd_floats = pl.partial_off + round_up(3 * pl.plane, 64);
    return pl;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static long long tile_blocks(const Shape& s) {
    const long long tasks = (long long)s.B * s.N * s.G;
    return (tasks + kWarpsPerBlock - 1) / kWarpsPerBlock;
}

template <int VEC>
static int run_forward(const FwdParams& p, Stream st) {
    const Shape& s = p.s;
    int rc = launch<FwdSummary<VEC, 4>>(p, tile_blocks(s), st);
    if (rc) return rc;
    CarryScan<false>::Params cp{p.sum, p.carry, p.state_in, nullptr, s};
    rc = launch<CarryScan<false>>(cp, (long long)s.B * ((s.C + 31) / 32), st);
    if (rc) return rc;
    return launch<FwdMaterialize<VEC, 4>>(p, tile_blocks(s), st);
}

template <int VEC>
static int run_backward(const BwdParams& p, Stream st) {
    const Shape& s = p.s;
    int rc = launch<BwdSummary<VEC, 4>>(p, tile_blocks(s), st);
    if (rc) return rc;
    CarryScan<true>::Params cp{p.sum, p.carry, p.grad_state_out, p.grad_state_in, s};
    rc = launch<CarryScan<true>>(cp, (long long)s.B * ((s.C + 31) / 32), st);
    if (rc) return rc;
    rc = launch<BwdMaterialize<VEC, 2>>(p, tile_blocks(s), st);
    if (rc) return rc;
    return launch<BwdReduce>(p, 3LL * ((s.C + 31) / 32), st);
}


// ---------------------------------------------------------------------------
// Single-pass forward: plan and launch.
// ---------------------------------------------------------------------------
struct SpPlan {
    SpShape s;
    long long tiles;
    size_t ctrl_words;               // header holding the error word
    size_t agg_off, incl_off;        // byte offsets into the workspace
    size_t bytes;
};

// Test build only: FIELDS_TILE_TICKET=1 hands tiles out through a counter (see stateful_entry).
#ifdef FIELDS_ALL_VARIANTS
static int tile_ticket_from_env() {
    const char* e = std::getenv("FIELDS_TILE_TICKET");
    return e && std::atoi(e) == 1 ? 1 : 0;
}
#else
static int tile_ticket_from_env() { return 0; }
#endif

static SpPlan make_sp_plan(int B, int L, int C, int tile_steps) {
    SpPlan pl{};
    pl.s.B = B; pl.s.L = L; pl.s.C = C;
    pl.s.NT = (L + tile_steps - 1) / tile_steps;
    pl.s.G = (C + kGroup - 1) / kGroup;
    pl.s.max_polls = kMaxPolls;
    pl.s.ticket = tile_ticket_from_env();
    pl.tiles = (long long)B * pl.s.G * pl.s.NT;
    pl.ctrl_words = kCtrlHeader;
    pl.agg_off = pl.ctrl_words * sizeof(unsigned);
    pl.incl_off = pl.agg_off + (size_t)pl.tiles * 4 * kGroup * sizeof(float);
    pl.bytes = pl.incl_off + (size_t)pl.tiles * 2 * kGroup * sizeof(float);
    return pl;
}


enum Algo { kAlgoAuto = 0, kAlgoThreePhase = 1, kAlgoSinglePass = 2, kAlgoWalk = 3 };

// The product library runs one kernel family: single pass wherever 128-bit accesses are
// possible, the scalar three-phase kernels otherwise. The measured alternatives (other tile
// shapes, the two-sweep forward, the direct-load and tile-resident backward, the chain walkers,
// the vectorised three-phase kernels, L2 prefetch) are compiled only into the test build
// (FIELDS_ALL_VARIANTS), which picks them per call from the environment:
//   FIELDS_READ_ALGO = three_phase | single_pass | walk, FIELDS_FWD_VARIANT, FIELDS_BWD_VARIANT,
//   FIELDS_READ_PREFETCH.
#ifdef FIELDS_ALL_VARIANTS
static Algo algo_from_env() {
    const char* e = std::getenv("FIELDS_READ_ALGO");
    if (!e) return kAlgoAuto;
    const std::string v(e);
    if (v == "three_phase") return kAlgoThreePhase;
    if (v == "single_pass") return kAlgoSinglePass;
    if (v == "walk") return kAlgoWalk;
    return kAlgoAuto;
}
#else
static Algo algo_from_env() { return kAlgoAuto; }
#endif

// Instantiations of the single-pass kernels. The first of each list is the default; the
// others are tuning alternatives selected with FIELDS_FWD_VARIANT / FIELDS_BWD_VARIANT.
//   forward  <steps per warp, warps, blocks per SM the registers must allow>
using FwdSp0 = FwdSinglePass<6, 8, 2>;        // tile 48 steps, 128 registers, no spills
#ifdef FIELDS_ALL_VARIANTS
using FwdSp1 = FwdSinglePass<4, 8, 2>;        // tile 32
//   two-sweep forward <steps per warp, warps, unroll, blocks per SM, ring slots>
using FwdSp2 = FwdTwoSweep<8, 4, 2, 4, 3>;    // tile 32, 16 warps per SM
//   staged: persistent blocks, the next tile's rows land in shared memory during the current tile
using FwdSp3 = FwdSinglePass<5, 8, 2, float, false, true>;  // tile 40, 74 KB per block
#endif
//   backward <steps per warp, warps, sweep-1 unroll, sweep-2 unroll, blocks per SM, rings, ring slots>
using BwdSp0 = BwdSinglePass<8, 4, 2, 1, 3, true, 3>;  // tile 32, 3-slot cp.async rings, 12 warps per SM
#ifdef FIELDS_ALL_VARIANTS
using BwdSp1 = BwdSinglePass<8, 4, 2, 1, 4>;           // direct loads, 16 warps per SM
#endif
//   backward with recomputed states <steps per warp, warps, steps per ring slot, blocks per SM, ring slots>
using BwdSp2 = BwdRecompute<8, 4, 1, 3, 2>;   // 73 KB per block, 12 warps per SM
//   tile resident in shared memory, recomputed states <steps per warp, warps, blocks per SM>
#ifdef FIELDS_ALL_VARIANTS
using BwdSp3 = BwdTileResident<4, 4, 3>;      // tile 16, 68 KB per block, 12 warps per SM
#endif
//   bfloat16 raw / read / grad_read / grad_raw (bits as uint16_t); state and arithmetic stay fp32
// The bfloat16 forward runs staged (persistent blocks, tickets one tile ahead, the next tile's
// rows landing in shared memory during the current tile): 40.6 us against 46.1 us for the
// one-tile-per-block form at 8 x 2,048 tokens. The fp32 forward does not (46.3 -> 51.6 us staged:
// it is within 10 % of a plain copy already and pays for 74 KB of shared-memory traffic per tile).
using FwdSpBf16 = FwdSinglePass<5, 8, 2, uint16_t, false, true>;
using FwdSpBf16Stats = FwdSinglePass<5, 8, 2, uint16_t, true, true>;  // also writes per-token sums of squares
// bfloat16 ring cells are half the size, so a 64-step tile (4 warps x 16 steps) still leaves room for
// four blocks per SM; measured 54.9 us against 59.7 us for the 32-step tile (and 71.5 us with
// 16-byte cells) on 8 x 2,048 tokens.
using BwdSpBf16 = BwdSinglePass<16, 4, 2, 1, 3, true, 3, uint16_t>;
constexpr int kSpMinTile = 32;     // smallest time tile of any forward instantiation above (workspace bound)
constexpr int kSpMinTileBwd = 16;  // same for the backward

#ifdef FIELDS_ALL_VARIANTS
static int variant_from_env(const char* name) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : 0;
}
#endif

// L2 prefetch of the next tile (test build: FIELDS_READ_PREFETCH = 1 for a distance of the
// number of resident blocks, a larger number for that distance). It gained 5 to 9 % on the
// batch-8 forward and lost as much on the backward and on long sequences: off in the product.
#ifdef FIELDS_ALL_VARIANTS
static int prefetch_from_env(int resident) {
    const char* e = std::getenv("FIELDS_READ_PREFETCH");
    const int v = e ? std::atoi(e) : 0;
    return v == 1 ? resident : (v > 1 ? v : 0);
}
#else
static int prefetch_from_env(int) { return 0; }
#endif

template <class K, typename IO = float>
static int run_forward_single_pass(const IO* raw, const float* tr, const float* ti,
                                   const float* gamma, const float* state_in, IO* read,
                                   float* state_out, void* workspace, int B, int L, int C,
                                   Stream st, float* sumsq = nullptr) {
    SpPlan pl = make_sp_plan(B, L, C, K::kTile);
    if constexpr (!K::kStaged) pl.s.prefetch = prefetch_from_env(resident_blocks<K>());
    char* ws = static_cast<char*>(workspace);
    unsigned* ctrl = reinterpret_cast<unsigned*>(ws);
    int rc = fill_unset(ws, pl.bytes, st);  // error word and every publication slot
    if (rc) return rc;
    SpFwdParamsT<IO> p{raw, tr, ti, gamma, state_in, read, state_out,
                       reinterpret_cast<float*>(ws + pl.agg_off),
                       reinterpret_cast<float*>(ws + pl.incl_off), ctrl, pl.s};
    p.sumsq = sumsq;
    if constexpr (K::kStaged) return launch_persistent<K>(p, pl.tiles, (long long)B * pl.s.G, st);
    else return launch_stateful<K>(p, pl.tiles, (long long)B * pl.s.G, st);
}

template <class K, typename IO = float>
static int run_backward_single_pass(const IO* raw, const float* tr, const float* ti,
                                    const float* gamma, const float* state_in, const IO* read,
                                    const IO* grad_read, const float* grad_state_out,
                                    IO* grad_raw, float* grad_tr, float* grad_ti,
                                    float* grad_gamma, float* grad_state_in, void* workspace,
                                    int B, int L, int C, Stream st,
                                    const float* states = nullptr) {
    SpPlan pl = make_sp_plan(B, L, C, K::kTile);
    pl.s.prefetch = prefetch_from_env(resident_blocks<K>());
    char* ws = static_cast<char*>(workspace);
    unsigned* ctrl = reinterpret_cast<unsigned*>(ws);
    int rc = fill_unset(ws, pl.bytes, st);
    if (rc) return rc;
    float* partial = reinterpret_cast<float*>(ws + pl.bytes);
    SpBwdParamsT<IO> p{raw, tr, ti, gamma, state_in, read, grad_read, grad_state_out, grad_raw,
                       grad_state_in, reinterpret_cast<float*>(ws + pl.agg_off),
                       reinterpret_cast<float*>(ws + pl.incl_off), ctrl, partial, pl.s};
    p.states = states;
    p.state_rows = L / kStateRowEvery;
    rc = launch_stateful<K>(p, pl.tiles, (long long)B * pl.s.G, st);
    if (rc) return rc;
    BwdParams rp{};
    rp.partial = partial;
    rp.grad_tr = grad_tr; rp.grad_ti = grad_ti; rp.grad_gamma = grad_gamma;
    rp.s = Shape{B, L, C, K::kTile, pl.s.NT, pl.s.G};
    return launch<BwdReduce>(rp, 3LL * ((C + 31) / 32), st);
}

static size_t sp_backward_bytes(int B, int L, int C, int tile_steps) {
    const SpPlan pl = make_sp_plan(B, L, C, tile_steps);
    return pl.bytes + (size_t)3 * B * pl.s.NT * C * sizeof(float);
}

#ifdef FIELDS_ALL_VARIANTS
// ---------------------------------------------------------------------------
// Chain walkers: one block per (batch row, 32 channels) walks the whole sequence, no
// inter-block communication, bitwise reproducible. Measured slower than the single-pass
// kernels on B200 at every shape tried (few warps per SM, scalar shared-memory traffic), so
// they run only on request (FIELDS_READ_ALGO=walk), e.g. when run-to-run identical bits
// matter more than speed. No workspace except one partial row per chain (backward).
// ---------------------------------------------------------------------------
using FwdWalker = FwdWalk<16, 8, 3>;   // tile 128 steps, 3 x 48 KB ring, 8 warps
using BwdWalker = BwdWalk<4, 8, 4>;    // tile 32 steps, 4 x 36 KB ring, 8 warps

template <class K>
static WalkShape walk_shape(int B, int L, int C) {
    return WalkShape{B, L, C, (L + K::kTile - 1) / K::kTile, (C + kLane - 1) / kLane};
}

static bool walk_wanted(int, int, Algo algo) { return algo == kAlgoWalk; }

#endif  // FIELDS_ALL_VARIANTS

// ---------------------------------------------------------------------------
// Sequence-sharded forward in one launch (field_span.cuh): plan.
// ---------------------------------------------------------------------------
using SpanFwd = FwdSpanSweep<2, 8, 2>;   // chunks of 2 steps (two in flight per warp), 8 warps, 2 blocks per SM
constexpr int kSpanMaxItems = 1024;       // runs per launch over all chains (unless there are more chains)

static long long span_item_bound(int B, int C) {
    const long long chains = (long long)B * ((C + kGroup - 1) / kGroup);
    return chains > kSpanMaxItems ? chains : kSpanMaxItems;
}

// Runs: as many per chain as the grid has blocks for, each a whole number of warp slices.
template <class K>
static SpanShape make_span_shape(int B, int L, int C, int grid) {
    SpanShape s{};
    s.B = B; s.L = L; s.C = C;
    s.G = (C + kGroup - 1) / kGroup;
    s.chains = B * s.G;
    long long want = grid / s.chains;
    const long long cap = span_item_bound(B, C) / s.chains;
    if (want > cap) want = cap;
    if (want > (L + K::kRunQuantum - 1) / K::kRunQuantum) want = (L + K::kRunQuantum - 1) / K::kRunQuantum;
    if (want < 1) want = 1;
    int steps = (int)((L + want - 1) / want);
    steps = (steps + K::kRunQuantum - 1) / K::kRunQuantum * K::kRunQuantum;
    s.run_steps = steps;
    s.R = (L + steps - 1) / steps;
    s.items = s.chains * s.R;
    return s;
}

// Bound of a device-side wait in polls: the caller's, or the library's default.
static unsigned poll_bound(unsigned max_polls) {
    return max_polls == 0 || max_polls > kMaxPolls ? kMaxPolls : max_polls;
}

// Mailbox = [slots of the exchange][board of the one-launch forward]. The board (the run maps
// of the owner's own kernel, 4 KB per run) is never written by a peer.
static size_t mailbox_slot_bytes(int P, int B, int C) {
    return round_up((size_t)2 * P * B * 4 * C * sizeof(MailPair), 256);
}
// counters (one word per chain), then the run maps of up to span_item_bound runs (2 KB each)
// (a counter word and, 256 bytes apart from one another, a ready word per chain)
// ... and, 64 words behind them, the two words of the device-resident epoch
static size_t board_epoch_offset(int B, int C) {
    return ((size_t)B * ((C + kGroup - 1) / kGroup) * 65 + 64) * sizeof(unsigned);
}
static size_t board_count_bytes(int B, int C) {
    return round_up(board_epoch_offset(B, C) + 64 * sizeof(unsigned), 256);
}
// Behind the board: the reduction region of fields_read_sum_over_ranks, [2][P][n_max] pairs.
static int mailbox_sum_capacity(int C) { return 3 * C + 64; }
static size_t mailbox_sum_bytes(int P, int C) {
    return round_up((size_t)2 * P * mailbox_sum_capacity(C) * sizeof(MailPair), 256);
}
static size_t mailbox_board_bytes(int B, int C) {
    return board_count_bytes(B, C) + (size_t)span_item_bound(B, C) * kGroup * 4 * sizeof(float);
}

// ---------------------------------------------------------------------------
// Built-in scratch for fields_read_forward_noalloc: one fixed buffer per GPU that
// has loaded this library, held until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = FIELDS_STATIC_SCRATCH_BYTES;

#ifdef FIELDS_HOST_EMU
alignas(256) static unsigned char g_static_scratch[kStaticScratchBytes];

static int static_scratch(float** out) {
    *out = reinterpret_cast<float*>(g_static_scratch);
    return FIELDS_OK;
}
#else
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static float* g_scratch_ptr[kMaxDevices] = {};

// In host code `g_static_scratch` is only a handle for the runtime, not an address a
// kernel may use: the device address is looked up once per device, with that device
// current, and cached.
static int static_scratch(float** out) {
    int dev = -1;
    int rc = check_cuda(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= kMaxDevices) return FIELDS_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        rc = check_cuda(cudaGetSymbolAddress(&p, g_static_scratch));
        if (rc) return rc;
        g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_ptr[dev];
    return FIELDS_OK;
}
#endif

}  // namespace fields

using namespace fields;

extern "C" {

const char* fields_status_string(int status) {
    switch (status) {
        case FIELDS_OK: return "ok";
        case FIELDS_ERR_ARGUMENT: return "invalid argument (null pointer or bad extent)";
        case FIELDS_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case FIELDS_ERR_LAUNCH: return "CUDA launch failed";
        case FIELDS_ERR_TIMEOUT: return "device-side wait timed out";
        case FIELDS_ERR_UNSUPPORTED: return "unsupported extent";
        case FIELDS_ERR_SCRATCH_LIMIT:
            return "extents need more scratch than the built-in static buffer holds";
        default: return "unknown status";
    }
}

int fields_read_version(void) { return 100; }

const char* fields_last_cuda_error(void) { return g_last_error; }

size_t fields_read_workspace_bytes(int B, int L, int C, int pass) {
    if (B <= 0 || L <= 0 || C <= 0) return 0;
    const Plan pl = make_plan(B, L, C, 1);
    const size_t floats = pass == FIELDS_PASS_BACKWARD ? pl.bwd_floats : pl.fwd_floats;
    size_t bytes = floats * sizeof(float);
    const size_t sp = pass == FIELDS_PASS_BACKWARD ? sp_backward_bytes(B, L, C, kSpMinTileBwd)
                                                   : make_sp_plan(B, L, C, kSpMinTile).bytes;
    return sp > bytes ? sp : bytes;
}

int fields_read_forward(const float* raw, const float* tr, const float* ti, const float* gamma,
                        const float* state_in, float* read, float* state_out, void* workspace,
                        size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    if (B == 0) return FIELDS_OK;
    if (!tr || !ti || !gamma) return FIELDS_ERR_ARGUMENT;
    if (L == 0) {
        // no steps: the state passes through unchanged
        if (state_out) {
            if (!state_in) return fill_zero(state_out, (size_t)B * 2 * C, st);
#ifdef FIELDS_HOST_EMU
            std::memcpy(state_out, state_in, (size_t)B * 2 * C * sizeof(float));
#else
            return check_cuda(cudaMemcpyAsync(state_out, state_in, (size_t)B * 2 * C * sizeof(float),
                                              cudaMemcpyDeviceToDevice, st));
#endif
        }
        return FIELDS_OK;
    }
    if (!raw || !read) return FIELDS_ERR_ARGUMENT;
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(read) && aligned16(tr) &&
                      aligned16(ti) && aligned16(gamma) && aligned16(state_in) &&
                      aligned16(state_out) && aligned16(workspace);
    const Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace || workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_FORWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    const Algo algo = algo_from_env();
#ifdef FIELDS_ALL_VARIANTS
    if (vec4 && walk_wanted(B, C, algo)) {
        WalkFwdParams wp{raw, tr, ti, gamma, state_in, read, state_out,
                         walk_shape<FwdWalker>(B, L, C)};
        return launch_walk<FwdWalker>(wp, (long long)B * wp.s.G, st);
    }
#endif
    if (vec4 && algo != kAlgoThreePhase) {
#define FIELDS_FWD_SP(K)                                                                      \
    return run_forward_single_pass<K>(raw, tr, ti, gamma, state_in, read, state_out, workspace, \
                                      B, L, C, st)
#ifdef FIELDS_ALL_VARIANTS
        switch (variant_from_env("FIELDS_FWD_VARIANT")) {
            case 1: FIELDS_FWD_SP(FwdSp1);
            case 2: FIELDS_FWD_SP(FwdSp2);
            case 3: FIELDS_FWD_SP(FwdSp3);
            default: FIELDS_FWD_SP(FwdSp0);
        }
#else
        FIELDS_FWD_SP(FwdSp0);
#endif
#undef FIELDS_FWD_SP
    }
    float* ws = static_cast<float*>(workspace);
    FwdParams p{raw, tr, ti, gamma, state_in, read, state_out,
                ws + pl.sum_off, ws + pl.carry_off, pl.s};
#ifdef FIELDS_ALL_VARIANTS
    if (vec4) return run_forward<4>(p, st);
#endif
    return run_forward<1>(p, st);
}

int fields_read_backward(const float* raw, const float* tr, const float* ti, const float* gamma,
                         const float* state_in, const float* read, const float* grad_read,
                         const float* grad_state_out, float* grad_raw, float* grad_tr,
                         float* grad_ti, float* grad_gamma, float* grad_state_in, void* workspace,
                         size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (!grad_tr || !grad_ti || !grad_gamma) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    if (B == 0 || L == 0) {
        // nothing depends on the parameters; the state gradient passes through
        int rc = fill_zero(grad_tr, C, st);
        if (!rc) rc = fill_zero(grad_ti, C, st);
        if (!rc) rc = fill_zero(grad_gamma, C, st);
        if (!rc && grad_state_in && B > 0) {
            if (!grad_state_out) {
                rc = fill_zero(grad_state_in, (size_t)B * 2 * C, st);
            } else {
#ifdef FIELDS_HOST_EMU
                std::memcpy(grad_state_in, grad_state_out, (size_t)B * 2 * C * sizeof(float));
#else
                rc = check_cuda(cudaMemcpyAsync(grad_state_in, grad_state_out,
                                                (size_t)B * 2 * C * sizeof(float),
                                                cudaMemcpyDeviceToDevice, st));
#endif
            }
        }
        return rc;
    }
    if (!raw || !tr || !ti || !gamma || !read || !grad_read || !grad_raw)
        return FIELDS_ERR_ARGUMENT;
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(read) && aligned16(grad_read) &&
                      aligned16(grad_raw) && aligned16(tr) && aligned16(ti) && aligned16(gamma) &&
                      aligned16(state_in) && aligned16(workspace);
    const Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace ||
        workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_BACKWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
#ifdef FIELDS_ALL_VARIANTS
    if (vec4 && walk_wanted(B, C, algo_from_env())) {
        float* partial = static_cast<float*>(workspace);
        WalkBwdParams wp{raw, tr, ti, gamma, state_in, read, grad_read, grad_state_out, grad_raw,
                         grad_state_in, partial, walk_shape<BwdWalker>(B, L, C)};
        int rc = launch_walk<BwdWalker>(wp, (long long)B * wp.s.G, st);
        if (rc) return rc;
        BwdParams rp{};
        rp.partial = partial;
        rp.grad_tr = grad_tr; rp.grad_ti = grad_ti; rp.grad_gamma = grad_gamma;
        rp.s = Shape{B, L, C, L, 1, wp.s.G};
        return launch<BwdReduce>(rp, 3LL * ((C + 31) / 32), st);
    }
#endif
    if (vec4 && algo_from_env() != kAlgoThreePhase) {
#define FIELDS_BWD_SP(K)                                                                        \
    return run_backward_single_pass<K>(raw, tr, ti, gamma, state_in, read, grad_read,          \
                                       grad_state_out, grad_raw, grad_tr, grad_ti, grad_gamma, \
                                       grad_state_in, workspace, B, L, C, st)
#ifdef FIELDS_ALL_VARIANTS
        switch (variant_from_env("FIELDS_BWD_VARIANT")) {
            case 1: FIELDS_BWD_SP(BwdSp1);
            case 2: FIELDS_BWD_SP(BwdSp2);
            case 3: FIELDS_BWD_SP(BwdSp3);
            default: FIELDS_BWD_SP(BwdSp0);
        }
#else
        FIELDS_BWD_SP(BwdSp0);
#endif
#undef FIELDS_BWD_SP
    }
    float* ws = static_cast<float*>(workspace);
    BwdParams p{raw, tr, ti, gamma, state_in, read, grad_read, grad_state_out, grad_raw,
                grad_state_in, ws + pl.sum_off, ws + pl.carry_off, ws + pl.partial_off,
                grad_tr, grad_ti, grad_gamma, pl.s};
#ifdef FIELDS_ALL_VARIANTS
    if (vec4) return run_backward<4>(p, st);
#endif
    return run_backward<1>(p, st);
}


int fields_read_state_rows(int L) { return L > 0 ? L / kStateRowEvery : 0; }

int fields_read_backward_from_states(const float* raw, const float* tr, const float* ti,
                                     const float* gamma, const float* state_in,
                                     const float* states, const float* grad_read,
                                     const float* grad_state_out, float* grad_raw, float* grad_tr,
                                     float* grad_ti, float* grad_gamma, float* grad_state_in,
                                     void* workspace, size_t workspace_bytes, int B, int L, int C,
                                     void* stream) {
    if (B <= 0 || L <= 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (!raw || !tr || !ti || !gamma || !grad_read || !grad_raw || !grad_tr || !grad_ti ||
        !grad_gamma)
        return FIELDS_ERR_ARGUMENT;
    if (!states && L > kStateRowEvery) return FIELDS_ERR_ARGUMENT;
    if (C % 4 != 0 || !aligned16(raw) || !aligned16(grad_read) || !aligned16(grad_raw) ||
        !aligned16(tr) || !aligned16(ti) || !aligned16(gamma) || !aligned16(state_in) ||
        !aligned16(states))
        return FIELDS_ERR_UNSUPPORTED;
    if (!workspace ||
        workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_BACKWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    // `read` is never dereferenced when the rows are given; a sequence of up to 8 steps needs no row
    return run_backward_single_pass<BwdSp2>(raw, tr, ti, gamma, state_in, (const float*)nullptr,
                                            grad_read, grad_state_out, grad_raw, grad_tr, grad_ti,
                                            grad_gamma, grad_state_in, workspace, B, L, C,
                                            reinterpret_cast<Stream>(stream), states);
}

size_t fields_read_static_scratch_bytes(void) { return kStaticScratchBytes; }

int fields_read_forward_noalloc(const float* raw, const float* tr, const float* ti,
                                const float* gamma, const float* state_in, float* read,
                                float* state_out, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    const size_t need = fields_read_workspace_bytes(B, L, C, FIELDS_PASS_FORWARD);
    if (need > kStaticScratchBytes) return FIELDS_ERR_SCRATCH_LIMIT;
    float* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc) return rc;
    // The forward kernels write every scratch word before they read it, so nothing has to
    // be cleared between calls.
    return fields_read_forward(raw, tr, ti, gamma, state_in, read, state_out, scratch,
                               kStaticScratchBytes, B, L, C, stream);
}


int fields_read_device_status(const void* workspace, void* stream) {
    if (!workspace) return FIELDS_ERR_ARGUMENT;
    int word = 0;
#ifdef FIELDS_HOST_EMU
    (void)stream;
    word = static_cast<const int*>(workspace)[0];
#else
    Stream st = reinterpret_cast<Stream>(stream);
    int rc = check_cuda(cudaMemcpyAsync(&word, static_cast<const int*>(workspace), sizeof(int),
                                        cudaMemcpyDeviceToHost, st));
    if (!rc) rc = check_cuda(cudaStreamSynchronize(st));
    if (rc) return rc;
#endif
    return word != -1 ? FIELDS_ERR_TIMEOUT : FIELDS_OK;
}


int fields_read_span_summary(const float* raw, const float* tr, const float* ti,
                             const float* gamma, float* summary, void* workspace,
                             size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !gamma || !summary) return FIELDS_ERR_ARGUMENT;
    if (L == 0) return FIELDS_ERR_ARGUMENT;  // an empty span has no summary to exchange
    Stream st = reinterpret_cast<Stream>(stream);
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(tr) && aligned16(ti) &&
                      aligned16(gamma) && aligned16(workspace);
    Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace || workspace_bytes < pl.fwd_floats * sizeof(float) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    float* ws = static_cast<float*>(workspace);
    FwdParams p{raw, tr, ti, gamma, nullptr, nullptr, nullptr, ws + pl.sum_off, ws + pl.carry_off,
                pl.s};
    int rc;
    if (vec4) {
        // 16 steps per warp, four warps per block: one map per 64 steps (never more maps than
        // the three-phase plan, whose workspace bound therefore still holds)
        using Stream4 = ChunkSummaryStream<2, 3, 4>;
        p.s.ts = 16;
        p.s.N = (L + 63) / 64;
        p.s.G = (C + 127) / 128;
        pl.s = p.s;
        rc = launch<Stream4>(p, (long long)B * p.s.N * p.s.G, st);
    } else {
        rc = launch<FwdSummary<1, 4>>(p, tile_blocks(pl.s), st);
    }
    if (rc) return rc;
    SpanCompose::Params cp{p.sum, summary, pl.s, 0};
    return launch<SpanCompose>(cp, (long long)B * ((C + 31) / 32), st);
}

int fields_read_span_summary_backward(const float* raw, const float* tr, const float* ti,
                                      const float* grad_read, float* summary, void* workspace,
                                      size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !grad_read || !summary) return FIELDS_ERR_ARGUMENT;
    if (L == 0) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(tr) && aligned16(ti) &&
                      aligned16(grad_read) && aligned16(workspace);
    const Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace || workspace_bytes < pl.bwd_floats * sizeof(float) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    float* ws = static_cast<float*>(workspace);
    BwdParams p{};
    p.raw = raw; p.tr = tr; p.ti = ti; p.grad_read = grad_read;
    p.sum = ws + pl.sum_off;
    p.s = pl.s;
    Shape cs = pl.s;
    int rc;
    if (vec4) {
        // as in fields_read_span_summary: 16 steps per warp, one map per 64 steps
        using Stream4 = ChunkDualSummaryStream<1, 3, 4>;  // 38 KB of shared memory per block
        p.s.ts = 16;
        p.s.N = (L + 63) / 64;
        p.s.G = (C + 127) / 128;
        cs = p.s;
        rc = launch<Stream4>(p, (long long)B * p.s.N * p.s.G, st);
    } else {
        rc = launch<BwdSummary<1, 4>>(p, tile_blocks(pl.s), st);
    }
    if (rc) return rc;
    SpanCompose::Params cp{p.sum, summary, cs, 1};
    return launch<SpanCompose>(cp, (long long)B * ((C + 31) / 32), st);
}

int fields_read_fold_summaries(const float* summaries, const float* state0, float* state,
                               int rank, int P, int B, int C, void* stream) {
    if (B < 0 || C <= 0 || P <= 0 || rank < 0 || rank >= P) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!summaries || !state) return FIELDS_ERR_ARGUMENT;
    FoldSummaries::Params p{summaries, state0, state, rank, P, B, C, 0};
    const long long n = (long long)B * C;
    return launch<FoldSummaries>(p, (n + FoldSummaries::kThreads - 1) / FoldSummaries::kThreads,
                                 reinterpret_cast<Stream>(stream));
}

int fields_read_fold_summaries_backward(const float* summaries, const float* carry_end, float* carry,
                                        int rank, int P, int B, int C, void* stream) {
    if (B < 0 || C <= 0 || P <= 0 || rank < 0 || rank >= P) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!summaries || !carry) return FIELDS_ERR_ARGUMENT;
    FoldSummaries::Params p{summaries, carry_end, carry, rank, P, B, C, 1};
    const long long n = (long long)B * C;
    return launch<FoldSummaries>(p, (n + FoldSummaries::kThreads - 1) / FoldSummaries::kThreads,
                                 reinterpret_cast<Stream>(stream));
}


}  // extern "C"

// ---------------------------------------------------------------------------
// Real-valued scan (field_scan.cuh): plan and launches.
// ---------------------------------------------------------------------------
static ScanShape make_scan_shape(int B, int L, int C, long long a_batch, long long a_step,
                                 int a_chan) {
    ScanShape s{};
    s.B = B; s.L = L; s.C = C;
    s.NT = (L + kScanChunk - 1) / kScanChunk;
    s.CG = (C + 31) / 32;
    s.a_batch = a_batch; s.a_step = a_step; s.a_chan = a_chan;
    return s;
}

static size_t scan_workspace_floats(int B, int L, int C) {
    return (size_t)3 * B * ((L + kScanChunk - 1) / kScanChunk) * C;
}

static int scan_check(const void* workspace, size_t workspace_bytes, int B, int L, int C,
                      long long a_batch, long long a_step, int a_chan) {
    if (a_chan != 0 && a_chan != 1) return FIELDS_ERR_ARGUMENT;
    if (a_batch < 0 || a_step < 0) return FIELDS_ERR_ARGUMENT;
    if (!workspace || workspace_bytes < scan_workspace_floats(B, L, C) * sizeof(float) ||
        (reinterpret_cast<uintptr_t>(workspace) & 15u))
        return FIELDS_ERR_WORKSPACE;
    return FIELDS_OK;
}

template <typename IO>
static int run_step(const IO* raw, const float* tr, const float* ti, const float* gamma,
                    float* state, IO* read, int B, int C, void* stream) {
    if (B < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !gamma || !state || !read) return FIELDS_ERR_ARGUMENT;
    typename DecodeStep<IO>::Params p{raw, tr, ti, gamma, state, read, B, C};
    const long long n = (long long)B * C;
    return launch<DecodeStep<IO>>(p, (n + DecodeStep<IO>::kThreads - 1) / DecodeStep<IO>::kThreads,
                                  reinterpret_cast<Stream>(stream));
}

extern "C" {

int fields_read_step(const float* raw, const float* tr, const float* ti, const float* gamma,
                     float* state, float* read, int B, int C, void* stream) {
    return run_step<float>(raw, tr, ti, gamma, state, read, B, C, stream);
}

int fields_read_step_bf16(const void* raw, const float* tr, const float* ti, const float* gamma,
                          float* state, void* read, int B, int C, void* stream) {
    return run_step<uint16_t>(static_cast<const uint16_t*>(raw), tr, ti, gamma, state,
                              static_cast<uint16_t*>(read), B, C, stream);
}


size_t fields_scan_workspace_bytes(int B, int L, int C) {
    if (B <= 0 || L <= 0 || C <= 0) return 0;
    return scan_workspace_floats(B, L, C) * sizeof(float);
}

int fields_scan_forward(const float* a, long long a_batch, long long a_step, int a_chan,
                        const float* drive, const float* state_in, float* states,
                        float* state_out, void* workspace, size_t workspace_bytes, int B, int L,
                        int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    if (B == 0) return FIELDS_OK;
    if (L == 0) {
        if (!state_out) return FIELDS_OK;
        if (!state_in) return fill_zero(state_out, (size_t)B * C, st);
#ifdef FIELDS_HOST_EMU
        std::memcpy(state_out, state_in, (size_t)B * C * sizeof(float));
        return FIELDS_OK;
#else
        return check_cuda(cudaMemcpyAsync(state_out, state_in, (size_t)B * C * sizeof(float),
                                          cudaMemcpyDeviceToDevice, st));
#endif
    }
    if (!a || !drive || !states) return FIELDS_ERR_ARGUMENT;
    int rc = scan_check(workspace, workspace_bytes, B, L, C, a_batch, a_step, a_chan);
    if (rc) return rc;
    const ScanShape s = make_scan_shape(B, L, C, a_batch, a_step, a_chan);
    float* ws = static_cast<float*>(workspace);
    const size_t plane = (size_t)B * s.NT * C;
    ScanFwdParams p{a, drive, state_in, states, state_out, ws, ws + plane, ws + 2 * plane, s};
    const long long chunk_blocks = (scan_items(s) + kScanWarps - 1) / kScanWarps;
    const long long chan_blocks = ((long long)B * C + ScanCarry::kThreads - 1) / ScanCarry::kThreads;
    rc = launch<ScanChunkMap>(p, chunk_blocks, st);
    if (!rc) rc = launch<ScanCarry>(p, chan_blocks, st);
    if (!rc) rc = launch<ScanEmit>(p, chunk_blocks, st);
    return rc;
}

int fields_scan_backward(const float* a, long long a_batch, long long a_step, int a_chan,
                         const float* states, const float* state_in, const float* grad_states,
                         const float* grad_state_out, float* grad_a, float* grad_drive,
                         float* grad_state_in, void* workspace, size_t workspace_bytes, int B,
                         int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    if (B == 0) return FIELDS_OK;
    if (L == 0) {
        if (!grad_state_in) return FIELDS_OK;
        if (!grad_state_out) return fill_zero(grad_state_in, (size_t)B * C, st);
#ifdef FIELDS_HOST_EMU
        std::memcpy(grad_state_in, grad_state_out, (size_t)B * C * sizeof(float));
        return FIELDS_OK;
#else
        return check_cuda(cudaMemcpyAsync(grad_state_in, grad_state_out,
                                          (size_t)B * C * sizeof(float), cudaMemcpyDeviceToDevice,
                                          st));
#endif
    }
    if (!a || !states || !grad_states || !grad_a || !grad_drive) return FIELDS_ERR_ARGUMENT;
    int rc = scan_check(workspace, workspace_bytes, B, L, C, a_batch, a_step, a_chan);
    if (rc) return rc;
    const ScanShape s = make_scan_shape(B, L, C, a_batch, a_step, a_chan);
    float* ws = static_cast<float*>(workspace);
    const size_t plane = (size_t)B * s.NT * C;
    ScanBwdParams p{a, states, state_in, grad_states, grad_state_out, grad_a, grad_drive,
                    grad_state_in, ws, ws + plane, ws + 2 * plane, s};
    const long long chunk_blocks = (scan_items(s) + kScanWarps - 1) / kScanWarps;
    const long long chan_blocks =
        ((long long)B * C + ScanCarryBwd::kThreads - 1) / ScanCarryBwd::kThreads;
    rc = launch<ScanChunkMapBwd>(p, chunk_blocks, st);
    if (!rc) rc = launch<ScanCarryBwd>(p, chan_blocks, st);
    if (!rc) rc = launch<ScanEmitBwd>(p, chunk_blocks, st);
    return rc;
}

int fields_read_selftest_wait(void* workspace, size_t workspace_bytes, unsigned max_polls,
                              void* stream) {
    // layout: [ctrl 256 B | agg 4 tiles | incl 4 tiles | out 128 x 2]
    const size_t agg_bytes = 4 * kGroup * 4 * sizeof(float), incl_bytes = 4 * kGroup * 2 * sizeof(float);
    const size_t need = kCtrlHeader * sizeof(unsigned) + agg_bytes + incl_bytes + kGroup * 2 * sizeof(float);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    if (max_polls == 0 || max_polls > kMaxPolls) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    char* ws = static_cast<char*>(workspace);
    int rc = fill_unset(ws, need, st);
    if (rc) return rc;
    float* agg = reinterpret_cast<float*>(ws + kCtrlHeader * sizeof(unsigned));
    float* incl = reinterpret_cast<float*>(ws + kCtrlHeader * sizeof(unsigned) + agg_bytes);
    float* out = reinterpret_cast<float*>(ws + kCtrlHeader * sizeof(unsigned) + agg_bytes + incl_bytes);
    WaitSelfTest::Params p{agg, incl, reinterpret_cast<unsigned*>(ws), out, max_polls};
    rc = launch<WaitSelfTest>(p, 1, st);
    if (rc) return rc;
    return fields_read_device_status(workspace, stream);
}


static bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

int fields_read_forward_bf16(const void* raw, const float* tr, const float* ti, const float* gamma,
                             const float* state_in, void* read, float* state_out, void* workspace,
                             size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0 || L == 0) {
        // nothing to scan: the fp32 entry point handles the state pass-through
        return fields_read_forward(nullptr, tr, ti, gamma, state_in, nullptr, state_out, workspace,
                                   workspace_bytes, B, 0, C, stream);
    }
    if (!raw || !read || !tr || !ti || !gamma) return FIELDS_ERR_ARGUMENT;
    if (C % 4 || !aligned8(raw) || !aligned8(read) || !aligned16(tr) || !aligned16(ti) ||
        !aligned16(gamma))
        return FIELDS_ERR_UNSUPPORTED;  // 64-bit accesses only: C % 4 == 0, 8-byte aligned rows
    if (!workspace || workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_FORWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    return run_forward_single_pass<FwdSpBf16, uint16_t>(
        static_cast<const uint16_t*>(raw), tr, ti, gamma, state_in, static_cast<uint16_t*>(read),
        state_out, workspace, B, L, C, reinterpret_cast<Stream>(stream));
}

int fields_read_forward_bf16_stats(const void* raw, const float* tr, const float* ti,
                                   const float* gamma, const float* state_in, void* read,
                                   float* sumsq, float* state_out, void* workspace,
                                   size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B <= 0 || L <= 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (!raw || !read || !sumsq || !tr || !ti || !gamma) return FIELDS_ERR_ARGUMENT;
    if (C % 4 || !aligned8(raw) || !aligned8(read) || !aligned16(tr) || !aligned16(ti) ||
        !aligned16(gamma))
        return FIELDS_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_FORWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    return run_forward_single_pass<FwdSpBf16Stats, uint16_t>(
        static_cast<const uint16_t*>(raw), tr, ti, gamma, state_in, static_cast<uint16_t*>(read),
        state_out, workspace, B, L, C, reinterpret_cast<Stream>(stream), sumsq);
}

int fields_read_backward_bf16(const void* raw, const float* tr, const float* ti, const float* gamma,
                              const float* state_in, const void* read, const void* grad_read,
                              const float* grad_state_out, void* grad_raw, float* grad_tr,
                              float* grad_ti, float* grad_gamma, float* grad_state_in,
                              void* workspace, size_t workspace_bytes, int B, int L, int C,
                              void* stream) {
    if (B < 0 || L < 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0 || L == 0)
        return fields_read_backward(nullptr, tr, ti, gamma, state_in, nullptr, nullptr, grad_state_out,
                                    nullptr, grad_tr, grad_ti, grad_gamma, grad_state_in, workspace,
                                    workspace_bytes, B, 0, C, stream);
    if (!raw || !read || !grad_read || !grad_raw || !tr || !ti || !gamma || !grad_tr || !grad_ti ||
        !grad_gamma)
        return FIELDS_ERR_ARGUMENT;
    if (C % 4 || !aligned8(raw) || !aligned8(read) || !aligned8(grad_read) || !aligned8(grad_raw) ||
        !aligned16(tr) || !aligned16(ti) || !aligned16(gamma) || !aligned16(state_in))
        return FIELDS_ERR_UNSUPPORTED;
    if (!workspace ||
        workspace_bytes < fields_read_workspace_bytes(B, L, C, FIELDS_PASS_BACKWARD) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    return run_backward_single_pass<BwdSpBf16, uint16_t>(
        static_cast<const uint16_t*>(raw), tr, ti, gamma, state_in,
        static_cast<const uint16_t*>(read), static_cast<const uint16_t*>(grad_read), grad_state_out,
        static_cast<uint16_t*>(grad_raw), grad_tr, grad_ti, grad_gamma, grad_state_in, workspace,
        B, L, C, reinterpret_cast<Stream>(stream));
}


size_t fields_read_mailbox_bytes(int P, int B, int C) {
    if (P <= 0 || B <= 0 || C <= 0) return 0;
    return mailbox_slot_bytes(P, B, C) + mailbox_board_bytes(B, C) + mailbox_sum_bytes(P, C);
}

int fields_read_sum_over_ranks(const float* values, float* out, int n, void* const* mailboxes,
                               unsigned* error_word, int rank, int P, unsigned epoch,
                               unsigned max_polls, int B, int C, void* stream) {
    if (B <= 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P || epoch == 0 || n < 0 ||
        n > mailbox_sum_capacity(C))
        return FIELDS_ERR_ARGUMENT;
    if (n == 0) return FIELDS_OK;
    if (!values || !out || !mailboxes || !error_word) return FIELDS_ERR_ARGUMENT;
    SumMailbox::Params p{};
    p.values = values; p.out = out; p.error = error_word;
    const size_t off = mailbox_slot_bytes(P, B, C) + mailbox_board_bytes(B, C);
    for (int r = 0; r < P; ++r) {
        if (!mailboxes[r] || (reinterpret_cast<uintptr_t>(mailboxes[r]) & 7u)) return FIELDS_ERR_ARGUMENT;
        p.region[r] = reinterpret_cast<MailPair*>(static_cast<char*>(mailboxes[r]) + off);
    }
    p.rank = rank; p.P = P; p.n = n; p.n_max = mailbox_sum_capacity(C);
    p.epoch = epoch; p.max_polls = poll_bound(max_polls);
    p.stages = 3;
#ifdef FIELDS_HOST_EMU
    p.stages = g_emu_span_stages & 3;  // the CPU tests run every rank's stores before any rank's wait
#endif
    return launch<SumMailbox>(p, (n + SumMailbox::kThreads - 1) / SumMailbox::kThreads,
                              reinterpret_cast<Stream>(stream));
}

int fields_read_forward_sharded(const float* raw, const float* tr, const float* ti,
                                const float* gamma, const float* state0, float* read,
                                float* state_out, float* summary, void* const* mailboxes,
                                unsigned* error_word, int rank, int P, unsigned epoch,
                                unsigned max_polls, int B, int L, int C, void* stream) {
    if (B < 0 || L <= 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P)
        return FIELDS_ERR_ARGUMENT;
#ifdef FIELDS_HOST_EMU
    if (epoch == 0) return FIELDS_ERR_ARGUMENT;  // the emulation runs a call as several partial launches
#endif
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !gamma || !read || !mailboxes || !error_word) return FIELDS_ERR_ARGUMENT;
    for (int r = 0; r < P; ++r)
        if (!mailboxes[r] || (reinterpret_cast<uintptr_t>(mailboxes[r]) & 255u)) return FIELDS_ERR_ARGUMENT;
    if (C % 4 != 0 || !aligned16(raw) || !aligned16(read) || !aligned16(tr) || !aligned16(ti) ||
        !aligned16(gamma))
        return FIELDS_ERR_UNSUPPORTED;
    Stream st = reinterpret_cast<Stream>(stream);
    const int grid_max = span_grid<SpanFwd>();
    if (grid_max <= 0) return FIELDS_ERR_LAUNCH;
    SpanFwdParams p{};
    p.raw = raw; p.tr = tr; p.ti = ti; p.gamma = gamma; p.state0 = state0;
    p.read = read; p.state_out = state_out; p.summary = summary;
    p.s = make_span_shape<SpanFwd>(B, L, C, grid_max);
    char* board = static_cast<char*>(mailboxes[rank]) + mailbox_slot_bytes(P, B, C);
    p.count = reinterpret_cast<unsigned*>(board);
    p.ready = p.count + p.s.chains;
    p.runmap = reinterpret_cast<float*>(board + board_count_bytes(B, C));
    p.emu_round = -1;
    p.error = error_word;
    for (int r = 0; r < P; ++r) p.mailbox[r] = static_cast<MailPair*>(mailboxes[r]);
    p.own = static_cast<const MailPair*>(mailboxes[rank]);
    p.rank = rank; p.P = P; p.epoch = epoch;
    // epoch 0: the epoch lives on the rank's board and the kernel advances it itself
    p.epoch_word = epoch == 0 ? reinterpret_cast<unsigned*>(board + board_epoch_offset(B, C)) : nullptr;
    p.max_polls = poll_bound(max_polls);
    p.stages = 3;
#ifdef FIELDS_HOST_EMU
    p.stages = g_emu_span_stages;  // the CPU tests run the ranks' first sweeps before any rank's wait
#endif
    const int grid = p.s.items < grid_max ? p.s.items : grid_max;
    return launch_span<SpanFwd>(p, grid, st);
}

int fields_read_span_summary_put(const float* raw, const float* tr, const float* ti,
                                 const float* gamma, void* const* mailboxes, float* summary,
                                 int rank, int P, unsigned epoch, void* workspace,
                                 size_t workspace_bytes, int B, int L, int C, void* stream) {
    if (B < 0 || L <= 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P || epoch == 0)
        return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !gamma || !mailboxes) return FIELDS_ERR_ARGUMENT;
    for (int r = 0; r < P; ++r)
        if (!mailboxes[r] || (reinterpret_cast<uintptr_t>(mailboxes[r]) & 7u)) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(tr) && aligned16(ti) &&
                      aligned16(gamma) && aligned16(workspace);
    Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace || workspace_bytes < pl.fwd_floats * sizeof(float) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    float* ws = static_cast<float*>(workspace);
    FwdParams p{raw, tr, ti, gamma, nullptr, nullptr, nullptr, ws + pl.sum_off, ws + pl.carry_off,
                pl.s};
    int rc;
    if (vec4) {
        using Stream4 = ChunkSummaryStream<2, 3, 4>;
        p.s.ts = 16;
        p.s.N = (L + 63) / 64;
        p.s.G = (C + 127) / 128;
        rc = launch<Stream4>(p, (long long)B * p.s.N * p.s.G, st);
    } else {
        rc = launch<FwdSummary<1, 4>>(p, tile_blocks(pl.s), st);
    }
    if (rc) return rc;
    PutSummary::Params pp{};
    pp.sum = p.sum;
    for (int r = 0; r < P; ++r) pp.mailbox[r] = static_cast<MailPair*>(mailboxes[r]);
    pp.summary = summary;
    pp.rank = rank; pp.P = P; pp.epoch = epoch;
    pp.s = p.s;
    pp.reverse = 0;
    return launch<PutSummary>(pp, (long long)B * ((C + 31) / 32), st);
}

int fields_read_span_summary_backward_put(const float* raw, const float* tr, const float* ti,
                                          const float* grad_read, void* const* mailboxes,
                                          float* summary, int rank, int P, unsigned epoch,
                                          void* workspace, size_t workspace_bytes, int B, int L,
                                          int C, void* stream) {
    if (B < 0 || L <= 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P || epoch == 0)
        return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !tr || !ti || !grad_read || !mailboxes) return FIELDS_ERR_ARGUMENT;
    for (int r = 0; r < P; ++r)
        if (!mailboxes[r] || (reinterpret_cast<uintptr_t>(mailboxes[r]) & 7u)) return FIELDS_ERR_ARGUMENT;
    Stream st = reinterpret_cast<Stream>(stream);
    const bool vec4 = C % 4 == 0 && aligned16(raw) && aligned16(tr) && aligned16(ti) &&
                      aligned16(grad_read) && aligned16(workspace);
    const Plan pl = make_plan(B, L, C, vec4 ? 4 : 1);
    if (!workspace || workspace_bytes < pl.bwd_floats * sizeof(float) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return FIELDS_ERR_WORKSPACE;
    float* ws = static_cast<float*>(workspace);
    BwdParams p{};
    p.raw = raw; p.tr = tr; p.ti = ti; p.grad_read = grad_read;
    p.sum = ws + pl.sum_off;
    p.s = pl.s;
    int rc;
    if (vec4) {
        using Stream4 = ChunkDualSummaryStream<1, 3, 4>;
        p.s.ts = 16;
        p.s.N = (L + 63) / 64;
        p.s.G = (C + 127) / 128;
        rc = launch<Stream4>(p, (long long)B * p.s.N * p.s.G, st);
    } else {
        rc = launch<BwdSummary<1, 4>>(p, tile_blocks(pl.s), st);
    }
    if (rc) return rc;
    PutSummary::Params pp{};
    pp.sum = p.sum;
    for (int r = 0; r < P; ++r) pp.mailbox[r] = static_cast<MailPair*>(mailboxes[r]);
    pp.summary = summary;
    pp.rank = rank; pp.P = P; pp.epoch = epoch;
    pp.s = p.s;
    pp.reverse = 1;
    return launch<PutSummary>(pp, (long long)B * ((C + 31) / 32), st);
}

int fields_read_fold_mailbox(const void* mailbox, const float* state0, float* state,
                             unsigned* error_word, int rank, int P, unsigned epoch,
                             unsigned max_polls, int B, int C, void* stream) {
    if (B < 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P || epoch == 0)
        return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!mailbox || !state || !error_word) return FIELDS_ERR_ARGUMENT;
    FoldMailbox::Params p{static_cast<const MailPair*>(mailbox), state0, state, error_word,
                          rank, P, B, C, epoch, poll_bound(max_polls), 0};
    const long long n = (long long)B * C;
    return launch<FoldMailbox>(p, (n + FoldMailbox::kThreads - 1) / FoldMailbox::kThreads,
                               reinterpret_cast<Stream>(stream));
}

int fields_read_fold_mailbox_backward(const void* mailbox, const float* carry_end, float* carry,
                                      unsigned* error_word, int rank, int P, unsigned epoch,
                                      unsigned max_polls, int B, int C, void* stream) {
    if (B < 0 || C <= 0 || P <= 0 || P > kMaxRanks || rank < 0 || rank >= P || epoch == 0)
        return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!mailbox || !carry || !error_word) return FIELDS_ERR_ARGUMENT;
    FoldMailbox::Params p{static_cast<const MailPair*>(mailbox), carry_end, carry, error_word,
                          rank, P, B, C, epoch, poll_bound(max_polls), 1};
    const long long n = (long long)B * C;
    return launch<FoldMailbox>(p, (n + FoldMailbox::kThreads - 1) / FoldMailbox::kThreads,
                               reinterpret_cast<Stream>(stream));
}

int fields_read_forward_bf16_tensor(const void* raw, const float* tr, const float* ti,
                                    const float* gamma, const float* state_in, void* read,
                                    float* state_out, unsigned* error_word, int B, int L, int C,
                                    void* stream) {
    if (B < 0 || L <= 0 || C <= 0) return FIELDS_ERR_ARGUMENT;
    if (B == 0) return FIELDS_OK;
    if (!raw || !read || !tr || !ti || !gamma || !error_word) return FIELDS_ERR_ARGUMENT;
    if (C % 4 || !aligned8(raw) || !aligned8(read)) return FIELDS_ERR_UNSUPPORTED;
    TensorFwdParams p{static_cast<const uint16_t*>(raw), tr, ti, gamma, state_in,
                      static_cast<uint16_t*>(read), state_out, error_word, B, L, C, kMaxPolls};
    const long long grid = (long long)B * ((C + kTcChannels - 1) / kTcChannels);
    if (grid > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
#ifdef FIELDS_HOST_EMU
    (void)stream;
    std::vector<double> store(kTcSmemBytesEmu / 8 + 2);
    for (long long block = 0; block < grid; ++block)
        FwdTensorChain::run_block_emu(p, (int)block, reinterpret_cast<char*>(store.data()));
    return FIELDS_OK;
#else
    static bool ready[64] = {};
    const int rc = allow_shared_memory(tensor_chain_entry, (size_t)kTcSmemBytes, ready);
    if (rc) return rc;
    return launch_on<TensorFwdParams>(tensor_chain_entry, (unsigned)grid, kTcThreads, kTcSmemBytes,
                                      reinterpret_cast<Stream>(stream), p);
#endif
}

#ifdef FIELDS_HOST_EMU
// Host emulation only: which parts fields_read_forward_sharded runs (bit 0: first sweep,
// bit 2: prefix maps and the store of the span's map into the mailboxes, bit 1: the same plus
// the wait and the second sweep), so a test can emulate several ranks in turn.
void fields_emu_span_stages(int stages) { g_emu_span_stages = stages; }
#endif

#ifndef FIELDS_HOST_EMU
size_t fields_mixer_epilogue_bias_rows(long long N) {
    return N > 0 ? (size_t)((N + kEpiRows - 1) / kEpiRows) : 0;
}

int fields_mixer_epilogue_forward(const float* x, const void* acc, const void* gate,
                                  const float* sumsq, const float* bias, const float* gate_bias,
                                  float* y, float eps, int features, long long N, int D,
                                  void* stream) {
    if (N < 0 || D <= 0 || features <= 0) return FIELDS_ERR_ARGUMENT;
    if (N == 0) return FIELDS_OK;
    if (!x || !acc || !gate || !sumsq || !bias || !y) return FIELDS_ERR_ARGUMENT;
    if (D % 4 || !aligned16(x) || !aligned16(y) || !aligned16(bias) || !aligned16(gate_bias) ||
        !aligned8(acc) || !aligned8(gate))
        return FIELDS_ERR_UNSUPPORTED;
    const long long blocks = (N + kEpiRows - 1) / kEpiRows;
    if (blocks > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    EpilogueParams p{x, static_cast<const uint16_t*>(acc), static_cast<const uint16_t*>(gate), sumsq,
                     bias, gate_bias, y, eps, 1.0f / (float)features, N, D};
    return launch_on<EpilogueParams>(epilogue_forward, (unsigned)blocks, kEpiThreads, 0,
                                     reinterpret_cast<Stream>(stream), p);
}

int fields_mixer_epilogue_backward(const float* grad_y, const void* acc, const void* gate,
                                   const float* sumsq, const float* bias, const float* gate_bias,
                                   void* grad_acc, void* grad_gate, float* grad_sumsq,
                                   float* grad_bias_rows, float* grad_gate_bias_rows, float eps,
                                   int features, long long N, int D, void* stream) {
    if (N < 0 || D <= 0 || features <= 0) return FIELDS_ERR_ARGUMENT;
    if (N == 0) return FIELDS_OK;
    if (!grad_y || !acc || !gate || !sumsq || !bias || !grad_acc || !grad_gate || !grad_sumsq ||
        !grad_bias_rows || (gate_bias && !grad_gate_bias_rows))
        return FIELDS_ERR_ARGUMENT;
    if (D % 4 || D > kEpiMaxD || !aligned16(grad_y) || !aligned16(bias) || !aligned16(gate_bias) ||
        !aligned16(grad_bias_rows) || !aligned16(grad_gate_bias_rows) || !aligned8(acc) ||
        !aligned8(gate) || !aligned8(grad_acc) || !aligned8(grad_gate))
        return FIELDS_ERR_UNSUPPORTED;
    const long long blocks = (N + kEpiRows - 1) / kEpiRows;
    if (blocks > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    EpilogueGradParams p{grad_y, static_cast<const uint16_t*>(acc),
                         static_cast<const uint16_t*>(gate), sumsq, bias, gate_bias,
                         static_cast<uint16_t*>(grad_acc), static_cast<uint16_t*>(grad_gate),
                         grad_sumsq, grad_bias_rows, grad_gate_bias_rows, eps,
                         1.0f / (float)features, N, D};
    return launch_on<EpilogueGradParams>(epilogue_backward, (unsigned)blocks, kEpiThreads, 0,
                                         reinterpret_cast<Stream>(stream), p);
}

int fields_read_norm_grad_combine(const void* grad_read, const void* read, const float* grad_sumsq,
                                  void* total, long long N, int F, void* stream) {
    if (N < 0 || F <= 0) return FIELDS_ERR_ARGUMENT;
    if (N == 0) return FIELDS_OK;
    if (!read || !grad_sumsq || !total) return FIELDS_ERR_ARGUMENT;
    if (F % 4 || !aligned8(grad_read) || !aligned8(read) || !aligned8(total))
        return FIELDS_ERR_UNSUPPORTED;
    const long long blocks = (N + kEpiRows - 1) / kEpiRows;
    if (blocks > 0x7fffffffLL) return FIELDS_ERR_UNSUPPORTED;
    NormGradParams p{static_cast<const uint16_t*>(grad_read), static_cast<const uint16_t*>(read),
                     grad_sumsq, static_cast<uint16_t*>(total), N, F};
    return launch_on<NormGradParams>(norm_grad_combine, (unsigned)blocks, kEpiThreads, 0,
                                     reinterpret_cast<Stream>(stream), p);
}
#endif  // FIELDS_HOST_EMU

}  // extern "C"
