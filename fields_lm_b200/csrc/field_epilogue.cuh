// Readout epilogue of the Field mixer: what follows the output projection once the RMS norm
// has been moved behind it (reference mixer: field_only_v4_chunked_triton_wiki100.py:1177-1179,
//   y = x + out_proj(read_norm(read)) * sigmoid(gate_proj(x)) ).
// With acc = read @ (W diag(w))^T (bfloat16, from the GEMM), g = gate_proj(x) (bfloat16) and
// sumsq = sum of squares of the token's 4C read values (from the recurrence kernel):
//   rstd = rsqrt(sumsq / features + eps)
//   y    = x + (acc * rstd + bias) * sigmoid(g + gate_bias)                      [N, D] fp32
// One pass over the four [N, D] tensors instead of seven elementwise library kernels, and one
// pass for all gradients:
//   go = grad_y * sigmoid(g)
//   grad_acc  = go * rstd                         (bfloat16)
//   grad_gate = grad_y * (acc * rstd + bias) * sigmoid(g) (1 - sigmoid(g))   (bfloat16)
//   grad_sumsq[n] = -0.5 rstd^3 / features * sum_d go * acc
//   grad_bias[d]  = sum_n go      (one partial row per block; the caller adds the rows)
//   grad_gate_bias[d] = sum_n grad_gate   (likewise; only when a gate bias is given)
//   grad_x = grad_y (the caller reuses the tensor)
// HBM-bound elementwise work: a thread owns four adjacent columns (16-byte fp32 and 8-byte bf16
// accesses), a warp one row at a time, a block kRows consecutive rows. Device only.
#pragma once

#include "field_math.cuh"

#ifndef FIELDS_HOST_EMU

namespace fields {

constexpr int kEpiThreads = 256;  // 8 warps; each thread owns 4 columns of every row it visits
constexpr int kEpiRows = 16;      // rows per block

struct EpilogueParams {
    const float* x;        // [N, D]
    const uint16_t* acc;   // [N, D] bf16
    const uint16_t* gate;  // [N, D] bf16
    const float* sumsq;    // [N]
    const float* bias;     // [D]
    const float* gate_bias;  // [D] or null: added to gate before the sigmoid
    float* y;              // [N, D]
    float eps, inv_features;
    long long N;
    int D;
};

struct EpilogueGradParams {
    const float* grad_y;   // [N, D]
    const uint16_t* acc;
    const uint16_t* gate;
    const float* sumsq;
    const float* bias;
    const float* gate_bias;     // [D] or null
    uint16_t* grad_acc;         // [N, D] bf16
    uint16_t* grad_gate;        // [N, D] bf16
    float* grad_sumsq;          // [N]
    float* grad_bias_rows;      // [blocks, D]
    float* grad_gate_bias_rows; // [blocks, D] or null: column sums of grad_gate
    float eps, inv_features;
    long long N;
    int D;
};

__device__ __forceinline__ float4 ldg4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// Rows are walked by whole blocks: all threads of the block take the same row, thread t the
// columns 4t, 4t + 4 * kEpiThreads, ... (D up to any multiple of 4).
__global__ void __launch_bounds__(kEpiThreads) epilogue_forward(const EpilogueParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long row0 = (long long)blockIdx.x * kEpiRows;
    for (int r = 0; r < kEpiRows; ++r) {
        const long long n = row0 + r;
        if (n >= p.N) return;
        const float rstd = rsqrtf(p.sumsq[n] * p.inv_features + p.eps);
        const size_t base = (size_t)n * p.D;
        for (int c = (int)threadIdx.x * 4; c < p.D; c += kEpiThreads * 4) {
            const float4 xv = __ldcs(reinterpret_cast<const float4*>(p.x + base + c));
            const Vec<4> a = io_load4_stream(p.acc + base + c);
            const Vec<4> g = io_load4_stream(p.gate + base + c);
            const float4 b = ldg4(p.bias + c);
            const float4 gb = p.gate_bias ? ldg4(p.gate_bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float bb[4] = {b.x, b.y, b.z, b.w};
            const float gbb[4] = {gb.x, gb.y, gb.z, gb.w};
            const float xx[4] = {xv.x, xv.y, xv.z, xv.w};
            float out[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                out[k] = xx[k] + (a.v[k] * rstd + bb[k]) * sigmoidf_fast(g.v[k] + gbb[k]);
            __stcs(reinterpret_cast<float4*>(p.y + base + c), make_float4(out[0], out[1], out[2], out[3]));
        }
    }
}

__global__ void __launch_bounds__(kEpiThreads) epilogue_backward(const EpilogueGradParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float warp_sums[kEpiRows][kEpiThreads / 32];
    const long long row0 = (long long)blockIdx.x * kEpiRows;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // column sums of go over this block's rows, kept per thread for the columns it owns
    constexpr int kMaxOwned = 4;  // D <= 4 * kEpiThreads * kMaxOwned / 4 columns per thread group
    float bias_acc[kMaxOwned][4], gate_acc[kMaxOwned][4];
#pragma unroll
    for (int j = 0; j < kMaxOwned; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) bias_acc[j][k] = gate_acc[j][k] = 0.0f;
    for (int r = 0; r < kEpiRows; ++r) {
        const long long n = row0 + r;
        if (n >= p.N) break;  // uniform over the block
        const float rstd = rsqrtf(p.sumsq[n] * p.inv_features + p.eps);
        const size_t base = (size_t)n * p.D;
        float dot = 0.0f;  // sum_d go * acc over this thread's columns
#pragma unroll
        for (int j = 0; j < kMaxOwned; ++j) {
            const int c = (int)threadIdx.x * 4 + j * kEpiThreads * 4;
            if (c < p.D) {
                const float4 gy = __ldcs(reinterpret_cast<const float4*>(p.grad_y + base + c));
                const Vec<4> a = io_load4_stream(p.acc + base + c);
                const Vec<4> g = io_load4_stream(p.gate + base + c);
                const float4 b = ldg4(p.bias + c);
                const float4 gb = p.gate_bias ? ldg4(p.gate_bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float bb[4] = {b.x, b.y, b.z, b.w};
                const float gbb[4] = {gb.x, gb.y, gb.z, gb.w};
                const float gg[4] = {gy.x, gy.y, gy.z, gy.w};
                Vec<4> ga, gt;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float s = sigmoidf_fast(g.v[k] + gbb[k]);
                    const float go = gg[k] * s;
                    ga.v[k] = go * rstd;
                    gt.v[k] = gg[k] * (a.v[k] * rstd + bb[k]) * (s - s * s);
                    dot += go * a.v[k];
                    bias_acc[j][k] += go;
                    gate_acc[j][k] += gt.v[k];
                }
                io_store4_stream(p.grad_acc + base + c, ga);
                io_store4_stream(p.grad_gate + base + c, gt);
            }
        }
        // row sum: lanes now, warps after the last row (one barrier per block, not two per row)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        if (lane == 0) warp_sums[r][warp] = dot;
    }
    __syncthreads();
    if (threadIdx.x < kEpiRows && row0 + threadIdx.x < p.N) {
        const long long n = row0 + threadIdx.x;
        const float rstd = rsqrtf(p.sumsq[n] * p.inv_features + p.eps);
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kEpiThreads / 32; ++w) total += warp_sums[threadIdx.x][w];
        p.grad_sumsq[n] = -0.5f * rstd * rstd * rstd * p.inv_features * total;
    }
#pragma unroll
    for (int j = 0; j < kMaxOwned; ++j) {
        const int c = (int)threadIdx.x * 4 + j * kEpiThreads * 4;
        if (c < p.D) {
            *reinterpret_cast<float4*>(p.grad_bias_rows + (size_t)blockIdx.x * p.D + c) =
                make_float4(bias_acc[j][0], bias_acc[j][1], bias_acc[j][2], bias_acc[j][3]);
            if (p.grad_gate_bias_rows)
                *reinterpret_cast<float4*>(p.grad_gate_bias_rows + (size_t)blockIdx.x * p.D + c) =
                    make_float4(gate_acc[j][0], gate_acc[j][1], gate_acc[j][2], gate_acc[j][3]);
        }
    }
}

// Gradient entering the recurrence when the norm statistics are an output too:
//   total = grad_read + 2 * grad_sumsq[token] * read          (all [N, F] bfloat16, fp32 arithmetic)
// d sumsq / d read = 2 read. grad_read may be null (then total = 2 grad_sumsq read). One pass.
struct NormGradParams {
    const uint16_t* grad_read;  // [N, F] bf16 or null
    const uint16_t* read;       // [N, F] bf16
    const float* grad_sumsq;    // [N]
    uint16_t* total;            // [N, F] bf16
    long long N;
    int F;
};

__global__ void __launch_bounds__(kEpiThreads) norm_grad_combine(const NormGradParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long row0 = (long long)blockIdx.x * kEpiRows;
    for (int r = 0; r < kEpiRows; ++r) {
        const long long n = row0 + r;
        if (n >= p.N) return;
        const float two_gs = 2.0f * p.grad_sumsq[n];
        const size_t base = (size_t)n * p.F;
        for (int c = (int)threadIdx.x * 4; c < p.F; c += kEpiThreads * 4) {
            const Vec<4> rd = io_load4_stream(p.read + base + c);
            Vec<4> out;
            if (p.grad_read) {
                const Vec<4> g = io_load4_stream(p.grad_read + base + c);
#pragma unroll
                for (int k = 0; k < 4; ++k) out.v[k] = g.v[k] + two_gs * rd.v[k];
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) out.v[k] = two_gs * rd.v[k];
            }
            io_store4_stream(p.total + base + c, out);
        }
    }
}

constexpr int kEpiMaxD = 4 * kEpiThreads * 4;  // 4,096 columns: four column groups per thread

}  // namespace fields

#endif  // FIELDS_HOST_EMU
