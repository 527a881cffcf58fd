// Inter-block publication for the single-pass kernels.
//
// A tile publishes two things per channel, each with ONE vector store into memory that
// was filled with the byte 0xFF before the launch:
//   aggregate  float4 (Re A, Im A, Re B, Im B)  the tile's affine map
//   inclusive  float2 (Re s, Im s)              the state after the tile
// A reader polls the words themselves: a component whose bits are still 0xFFFFFFFF has
// not arrived. No flag, no fence and no ordering between the stores is needed, and a
// look-back step costs one L2 round trip. 0xFFFFFFFF is a NaN pattern that arithmetic
// never produces (hardware NaNs are 0x7FFFFFFF), so genuine data cannot be mistaken for
// "not yet written"; if it ever were, the bounded wait below reports it instead of hanging.
//
// Device versions are volatile (L2-coherent) vector accesses. Host versions
// (FIELDS_HOST_EMU) are plain accesses: the emulation runs one thread at a time and
// treats "not yet written" as an error at once.
#pragma once

#include "field_math.cuh"

namespace fields {

// Upper bound on polls of one slot: a poll is an L2 round trip plus a short sleep (well
// under a microsecond), so the bound is roughly a second. A wait that reaches it records
// an error, poisons its result with NaN and returns: the kernel always terminates.
constexpr unsigned kMaxPolls = 1u << 21;
constexpr unsigned kUnsetBits = 0xFFFFFFFFu;
constexpr int kUnsetByte = 0xFF;

FL_HD bool is_unset(float x) {
#if FL_DEVICE_CODE
    return __float_as_uint(x) == kUnsetBits;
#else
    unsigned u;
    std::memcpy(&u, &x, 4);
    return u == kUnsetBits;
#endif
}

struct Pub4 { float x, y, z, w; };
struct Pub2 { float x, y; };

FL_HD void publish4(float* p, float x, float y, float z, float w) {
#if FL_DEVICE_CODE
    asm volatile("st.volatile.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x), "f"(y),
                 "f"(z), "f"(w)
                 : "memory");
#else
    p[0] = x; p[1] = y; p[2] = z; p[3] = w;
#endif
}

FL_HD void publish2(float* p, float x, float y) {
#if FL_DEVICE_CODE
    asm volatile("st.volatile.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(x), "f"(y) : "memory");
#else
    p[0] = x; p[1] = y;
#endif
}

FL_HD Pub4 peek4(const float* p) {
    Pub4 r;
#if FL_DEVICE_CODE
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
                 : "l"(p)
                 : "memory");
#else
    r.x = p[0]; r.y = p[1]; r.z = p[2]; r.w = p[3];
#endif
    return r;
}

FL_HD Pub2 peek2(const float* p) {
    Pub2 r;
#if FL_DEVICE_CODE
    asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "l"(p) : "memory");
#else
    r.x = p[0]; r.y = p[1];
#endif
    return r;
}

// ---------------------------------------------------------------------------
// Asynchronous 16-byte global -> shared copies.
// ---------------------------------------------------------------------------
FL_HD void async_copy16(float* smem_dst, const float* gmem_src) {
#if FL_DEVICE_CODE
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(gmem_src)
                 : "memory");
#else
    std::memcpy(smem_dst, gmem_src, 16);
#endif
}

// Four elements (16 bytes of float, 8 bytes of bf16) into a shared-memory cell aligned to its size.
FL_HD void async_copy4(float* cell, const float* src) { async_copy16(cell, src); }

FL_HD void async_copy4(float* cell, const uint16_t* src) {
#if FL_DEVICE_CODE
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(cell);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(saddr), "l"(src) : "memory");
#else
    std::memcpy(cell, src, 8);
#endif
}

// Reads back a cell filled by async_copy4 from a source of element type IO.
template <typename IO>
FL_HD Vec<4> cell_load4(const float* cell) {
    if constexpr (sizeof(IO) == 4) {
        return vec_load<4>(cell);
    } else {
#if FL_DEVICE_CODE
        const uint2 w = *reinterpret_cast<const uint2*>(cell);
        return bf16x4_unpack(w.x, w.y);
#else
        uint32_t w[2];
        std::memcpy(w, cell, 8);
        return bf16x4_unpack(w[0], w[1]);
#endif
    }
}

FL_HD void async_commit() {
#if FL_DEVICE_CODE
    asm volatile("cp.async.commit_group;" ::: "memory");
#endif
}

template <int N>
FL_HD void async_wait_pending() {
#if FL_DEVICE_CODE
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
#endif
}

// Waits until at most `n` of this thread's copy groups are still pending (n known only at
// run time; the instruction wants an immediate).
FL_HD void async_wait_pending_dyn(int n) {
#if FL_DEVICE_CODE
    switch (n) {
        case 0: async_wait_pending<0>(); break;
        case 1: async_wait_pending<1>(); break;
        case 2: async_wait_pending<2>(); break;
        case 3: async_wait_pending<3>(); break;
        case 4: async_wait_pending<4>(); break;
        case 5: async_wait_pending<5>(); break;
        case 6: async_wait_pending<6>(); break;
        default: async_wait_pending<7>(); break;
    }
#else
    (void)n;
#endif
}

// Asks the memory system to bring one 128-byte line into L2 (no register, no wait).
FL_HD void prefetch_l2(const void* p) {
#if FL_DEVICE_CODE
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
#else
    (void)p;
#endif
}

FL_HD void backoff(unsigned polls) {
#if FL_DEVICE_CODE
    __nanosleep(polls < 32 ? 32 : 256);
#else
    (void)polls;
#endif
}

// The error word starts as 0xFFFFFFFF (same fill as the slots); any other value is an error.
FL_HD void error_record(unsigned* error, unsigned code) {
#if FL_DEVICE_CODE
    atomicMin(error, code);
#else
    if (*error > code) *error = code;
#endif
}

// Walks back from tile n-1 of a chain until a tile with a published end state is met,
// composing the aggregates of the tiles in between, and returns the state entering tile n.
// Four predecessors are fetched per round trip and consumed in order as far as they are ready.
//   agg  [tile][128][4], incl [tile][128][2]: slots of this chain start at `chain_base`.
// `thread` is the channel inside the 128-channel group. n must be > 0.
FL_HD void look_back(const float* agg, const float* incl, long long chain_base, int n, int thread,
                     unsigned* error, unsigned max_polls, float& sr, float& si) {
    constexpr int W = 4;           // predecessors fetched per round trip (6 and 8 measured slower: registers)
    Affine M = affine_identity();  // maps of the tiles between the one met and tile n
    int k = n - 1;                 // nearest tile not yet folded into M
    unsigned polls = 0;
    for (;;) {
        Pub2 s[W];
        Pub4 a[W];
#pragma unroll
        for (int j = 0; j < W; ++j) {
            if (k - j >= 0) {
                const long long slot = (chain_base + k - j) * 128 + thread;
                s[j] = peek2(incl + slot * 2);
                a[j] = peek4(agg + slot * 4);
            }
        }
        int used = 0;
#pragma unroll
        for (int j = 0; j < W; ++j) {
            if (used != j || k - j < 0) continue;  // stop at the first slot that is not ready
            if (!is_unset(s[j].x) && !is_unset(s[j].y)) {
                sr = s[j].x;
                si = s[j].y;
                affine_apply(M, sr, si);
                return;
            }
            if (k - j > 0 && !is_unset(a[j].x) && !is_unset(a[j].y) && !is_unset(a[j].z) &&
                !is_unset(a[j].w)) {
                // first a, then M
                M = affine_then(Affine{a[j].x, a[j].y, a[j].z, a[j].w}, M.ar, M.ai, M.br, M.bi);
                used = j + 1;
            }
        }
        if (used > 0) {
            k -= used;
            polls = 0;
            continue;
        }
#if FL_DEVICE_CODE
        if (++polls < max_polls) {
            backoff(polls);
            continue;
        }
#else
        (void)max_polls;
        (void)polls;
#endif
        error_record(error, 1u);
        sr = si = nanf("");
        return;
    }
}

}  // namespace fields
