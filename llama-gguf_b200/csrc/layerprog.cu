// layerprog.cu — layer-program models: a decoder given as a list of layers, each with its own token mixer (see the block
// "layer-program models" of include/llama_b200.h for the mechanisms and their parameters).
//
// A STEP is a batch of token runs, each continuing one sequence slot.  All rows of a step share the weight passes (one GEMM per
// fused projection over all rows); the mixers work per (run, head) from the slot's cache / state, so a prompt, a portion of a
// prompt and a single decoded token are the same code with another run length.  Row r of a step knows its run and its position
// through small device arrays written once per step.
//
// Precision: the residual stream, norms, softmax, gates, decays, unit norms and every recurrent state are f32 in both compute
// modes.  B200_COMPUTE_BF16 keeps the matrices and the GEMM operands in bf16 (f32 accumulation, f32 results);
// B200_COMPUTE_F32 keeps them in f32 and multiplies with FMA on the CUDA cores (no reduced-precision matrix mode).
#include "layerprog.h"

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

namespace {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------------------------------------ device helpers
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float logsigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// Per-step row / run tables (device).  Row r belongs to run row_run[r] and sits at position row_pos[r] of its sequence; run s covers
// rows [run_start[s], run_start[s + 1]), starts at position run_pos0[s] and owns the cache run_kv[s] and the state run_rec[s].
struct StepMeta {
    const int* tok;
    const int* row_run;
    const int* row_pos;
    const int* run_start;
    const int* run_pos0;
    uint8_t* const* run_kv;
    uint8_t* const* run_rec;
    const int* want;
};

// ------------------------------------------------------------------------------------------------ embedding
// x[r] = table[token] * scale (+ sinusoidal position vector: entry 2i = sin(p w_i), entry 2i + 1 = cos(p w_i), w_i = 10000^(-2i/width)).
// The angle and its sine are evaluated in double: at positions in the thousands an f32 angle alone is off by 1e-4.
template <typename T>
__global__ void lp_embed_kernel(StepMeta sm, const T* __restrict__ table, const double* __restrict__ inv_freq, float* __restrict__ x,
                                int width, float scale, int sinusoid) {
    const int r = blockIdx.x;
    const T* row = table + (size_t)sm.tok[r] * width;
    const double p = (double)sm.row_pos[r];
    for (int i = threadIdx.x; i < (width + 1) / 2; i += blockDim.x) {
        float s = 0.0f, c = 0.0f;
        if (sinusoid) {
            double ds, dc;
            sincos(p * inv_freq[i], &ds, &dc);
            s = (float)ds;
            c = (float)dc;
        }
        x[(size_t)r * width + 2 * i] = to_f(row[2 * i]) * scale + s;
        if (2 * i + 1 < width) x[(size_t)r * width + 2 * i + 1] = to_f(row[2 * i + 1]) * scale + c;
    }
}

// ------------------------------------------------------------------------------------------------ RMS norm
// out[b] = x[src] / sqrt(mean(x[src]^2) + eps) * w, src = gather ? gather[b] : b.  add != null: x[src] += add first (stored back):
// the per-pass step vector of a repeated layer range.  center = 1: the layer norm, (x - mean) / sqrt(mean((x - mean)^2) + eps) * w
// (the mean in a pass of its own).  One block per row.
template <typename OutT>
__global__ void lp_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ add, const float* __restrict__ w, OutT* __restrict__ out,
                                  const int* __restrict__ gather, int width, float eps, int center) {
    const int b = blockIdx.x;
    const int r = gather ? gather[b] : b;
    float* xr = x + (size_t)r * width;
    __shared__ float red[34];
    float mean = 0.0f;
    if (center) {
        float t = 0.0f;
        for (int c = threadIdx.x; c < width; c += blockDim.x) t += xr[c] + (add ? add[c] : 0.0f);
        t = wsum(t);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
        __syncthreads();
        if (threadIdx.x < 32) {
            float u = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
            u = wsum(u);
            if (threadIdx.x == 0) red[33] = u / (float)width;
        }
        __syncthreads();
        mean = red[33];
    }
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = xr[c];
        if (add) {
            v += add[c];
            xr[c] = v;
        }
        ss += (v - mean) * (v - mean);
    }
    ss = wsum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
        t = wsum(t);
        if (threadIdx.x == 0) red[32] = 1.0f / sqrtf(t / (float)width + eps);
    }
    __syncthreads();
    const float inv = red[32];
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)b * width + c] = from_f<OutT>((xr[c] - mean) * inv * w[c]);
}

// ------------------------------------------------------------------------------------------------ GEMM (CUDA cores)
// Y[r][n] = epi(alpha * sum_k X[r][k] * W[n][k] + bias[n]); products of the stored operand values in f32, f32 accumulation
// (bias: f32 per output column, or null).
enum { EPI_STORE = 0, EPI_ADD = 1, EPI_RELU2 = 2, EPI_GELU = 3, EPI_COUNT = 4 };
__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f)); }
template <typename T, int EPI>
__device__ __forceinline__ void epi_store(void* Y, size_t idx, float v) {
    if (EPI == EPI_STORE) reinterpret_cast<float*>(Y)[idx] = v;
    else if (EPI == EPI_ADD) reinterpret_cast<float*>(Y)[idx] += v;
    else if (EPI == EPI_GELU) reinterpret_cast<T*>(Y)[idx] = from_f<T>(gelu_erf_f(v));
    else {
        const float z = fmaxf(v, 0.0f);
        reinterpret_cast<T*>(Y)[idx] = from_f<T>(z * z);
    }
}

// the output row `off` elements on (f32 for the store / add epilogues, the compute type for the activations)
template <typename T, int EPI>
__device__ __forceinline__ void* seg_rows(void* Y, size_t off) {
    return (EPI == EPI_RELU2 || EPI == EPI_GELU) ? (void*)(reinterpret_cast<T*>(Y) + off) : (void*)(reinterpret_cast<float*>(Y) + off);
}
// Products batched over grid.z without row segments (the heads of a mixer): group z reads X and writes Y `xz` / `yz` elements on
struct ZStride {
    size_t x, y;
};
constexpr int GB = 64, GK = 16;
template <typename T, int EPI>
__global__ void __launch_bounds__(256) lp_gemm_kernel(const T* __restrict__ X, int ldx, const T* __restrict__ W, int ldw, void* __restrict__ Y,
                                                      int ldy, int R, int N, int K, float alpha, const int* __restrict__ seg, size_t w_zstride, ZStride zs,
                                                      const float* __restrict__ bias) {
    __shared__ float As[GK][GB + 4];
    __shared__ float Bs[GK][GB + 4];
    if (!seg && gridDim.z > 1) {
        W += blockIdx.z * w_zstride;
        X += blockIdx.z * zs.x;
        Y = seg_rows<T, EPI>(Y, blockIdx.z * zs.y);
    }
    if (seg) {   // grid.z = group: rows [seg[0], seg[0] + seg[1]) of X and Y, known on the device only (R is the launch's upper bound),
                 // against the group's own weight matrix
        seg += 2 * blockIdx.z;
        W += blockIdx.z * w_zstride;
        X += (size_t)seg[0] * ldx;
        Y = seg_rows<T, EPI>(Y, (size_t)seg[0] * ldy);
        R = seg[1];
        if ((int)blockIdx.y * GB >= R) return;
    }
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int r0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int k = k0 + lk + i;
            const int r = r0 + lr, n = n0 + lr;
            As[lk + i][lr] = (r < R && k < K) ? to_f(X[(size_t)r * ldx + k]) : 0.0f;
            Bs[lk + i][lr] = (n < N && k < K) ? to_f(W[(size_t)n * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; k++) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = r0 + ty * 4 + i;
        if (r >= R) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) epi_store<T, EPI>(Y, (size_t)r * ldy + n, alpha * acc[i][j] + (bias ? bias[n] : 0.0f));
        }
    }
}

// ------------------------------------------------------------------------------------------------ GEMM (tcgen05 / TMEM, bf16)
// Y[t][n] = epi(alpha * sum_k X[t][k] W[n][k]) for many rows: one CTA of 128 threads per (128 weight rows, TN tokens) tile, the f32
// accumulator in TMEM (TN columns x 128 lanes).  Per K step of 64 elements (128 bytes of bf16 = one row of a 128-byte swizzle
// atom) the threads copy the weight rows and the activation rows with 16-byte cp.async into K-major SWIZZLE_128B tiles (chunk c of
// row r lands at chunk c ^ (r & 7)); TC_STAGES such stages are in flight.  When a stage has landed: fence.proxy.async, barrier,
// and one thread issues 4 x tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = TN, K = 16, bf16 operands) and commits them to the
// stage's mbarrier; a stage is refilled when that commit has arrived.  Epilogue: warp w reads TMEM lanes 32w .. 32w + 31 (= weight
// rows) 32 token columns at a time; a warp's stores of one token are 32 consecutive outputs.  Every mbarrier wait is bounded: a
// wait that gives up sets *err and the CTA drains its copies, frees its TMEM columns and returns.
constexpr int TC_M = 128, TC_K = 64, TC_STAGES = 4;
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// K-major SWIZZLE_128B shared-memory matrix descriptor: start >> 4, LBO (unused) = 1, SBO = 1024 bytes between 8-row groups,
// version 1 at bit 46, layout SWIZZLE_128B = 2 at bit 61
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: D = f32 (bits 4-5 = 1), A = B = bf16 (1 at bits 7 and 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__device__ __forceinline__ uint32_t tc_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    const long long t0 = clock64();
    while (!ok) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (!ok && clock64() - t0 > 2000000000LL) return false;
    }
    return true;
}
__device__ __forceinline__ uint32_t tc_sw128(int r, int c) {
    return (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u + (uint32_t)((c ^ (r & 7)) << 4);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t bytes) {   // bytes = 16, or 0 for a zero chunk
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

template <int TN, int EPI>
__global__ void __launch_bounds__(128) lp_gemm_tc_kernel(const bf16* __restrict__ X, int ldx, const bf16* __restrict__ W, int ldw,
                                                         void* __restrict__ Y, int ldy, int R, int N, int K, float alpha, int* err,
                                                         const int* __restrict__ seg, size_t w_zstride, ZStride zs, const float* __restrict__ bias) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    if (!seg && gridDim.z > 1) {
        W += blockIdx.z * w_zstride;
        X += blockIdx.z * zs.x;
        Y = seg_rows<bf16, EPI>(Y, blockIdx.z * zs.y);
    }
    if (seg) {   // grid.z = group: rows [seg[0], seg[0] + seg[1]) of X and Y, known on the device only, against the group's own weight
                 // matrix; a CTA beyond the rows leaves before it holds anything
        seg += 2 * blockIdx.z;
        W += blockIdx.z * w_zstride;
        X += (size_t)seg[0] * ldx;
        Y = seg_rows<bf16, EPI>(Y, (size_t)seg[0] * ldy);
        R = seg[1];
        if ((int)blockIdx.y * TN >= R) return;
    }
    __shared__ __align__(8) unsigned long long s_bar[TC_STAGES];
    __shared__ uint32_t s_tmem;
    constexpr int kStage = (TC_M + TN) * 128;
    uint8_t* base = tc_smem + ((1024u - (smem_u32(tc_smem) & 1023u)) & 1023u);   // the swizzle is on absolute address bits
    const int tid = threadIdx.x, warp = tid >> 5;
    const int n0 = blockIdx.x * TC_M, t0 = blockIdx.y * TN;
    const uint32_t bar = smem_u32(&s_bar[0]);
    constexpr int kCols = TN < 32 ? 32 : TN;
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < TC_STAGES; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar + 8u * i) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "n"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const uint32_t idesc = tc_idesc(TC_M, TN);
    const int steps = (K + TC_K - 1) / TC_K;
    // copies of K step `st` into its stage: 8 chunks per row, (128 + TN) rows, spread over the 128 threads
    auto load = [&](int st) {
        uint8_t* tA = base + (st % TC_STAGES) * kStage;
        uint8_t* tB = tA + TC_M * 128;
        const int k0 = st * TC_K;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = tid + u * 128, r = i >> 3, c = i & 7, n = n0 + r, k = k0 + 8 * c;
            const bool in = n < N && k < K;
            cp_async16(smem_u32(tA + tc_sw128(r, c)), in ? (const void*)(W + (size_t)n * ldw + k) : (const void*)W, in ? 16u : 0u);
        }
#pragma unroll
        for (int u = 0; u < TN / 16; u++) {
            const int i = tid + u * 128, r = i >> 3, c = i & 7, t = t0 + r, k = k0 + 8 * c;
            const bool in = t < R && k < K;
            cp_async16(smem_u32(tB + tc_sw128(r, c)), in ? (const void*)(X + (size_t)t * ldx + k) : (const void*)X, in ? 16u : 0u);
        }
    };
    for (int st = 0; st < TC_STAGES - 1; st++) {
        if (st < steps) load(st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    bool alive = true;
    for (int it = 0; it < steps; it++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TC_STAGES - 2) : "memory");   // this thread's copies of step `it` have landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");               // generic-proxy writes -> visible to the tensor core
        __syncthreads();
        if (tid == 0 && alive) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint8_t* tA = base + (it % TC_STAGES) * kStage;
            const uint64_t da = tc_desc(smem_u32(tA)), db = tc_desc(smem_u32(tA + TC_M * 128));
#pragma unroll
            for (int kk = 0; kk < TC_K / 16; kk++) {   // 16 bf16 = 32 bytes along the swizzled row: start address + 2
                const uint32_t accum = (it > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem),
                    "l"(da + (uint64_t)(2 * kk)), "l"(db + (uint64_t)(2 * kk)), "r"(idesc), "r"(accum)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar + 8u * (it % TC_STAGES)) : "memory");
        }
        // refill the stage that step it - 1 read: its MMAs must be done (they run while the MMAs of step `it` wait in the queue)
        const int nx = it + TC_STAGES - 1;
        if (nx < steps) {
            if (it >= 1 && alive) {
                const int ps = (it - 1) % TC_STAGES;
                if (!tc_wait(bar + 8u * ps, (uint32_t)(((it - 1) / TC_STAGES) & 1))) {
                    alive = false;
                    if (err) atomicExch(err, 1);
                }
            }
            if (alive) load(nx);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (alive && steps > 0 && !tc_wait(bar + 8u * ((steps - 1) % TC_STAGES), (uint32_t)(((steps - 1) / TC_STAGES) & 1))) {
        alive = false;
        if (err) atomicExch(err, 2);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n = n0 + tid;
    const float bn = (bias && n < N) ? bias[n] : 0.0f;
    if (alive) {
#pragma unroll 1
        for (int c0 = 0; c0 < TN; c0 += 32) {
            if (t0 + c0 >= R) break;   // CTA-uniform
            uint32_t v[32];
            const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                  "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                  "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                  "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (n < N) {
#pragma unroll
                for (int c = 0; c < 32; c++) {
                    const int t = t0 + c0 + c;
                    if (t < R) epi_store<bf16, EPI>(Y, (size_t)t * ldy + n, alpha * __uint_as_float(v[c]) + bn);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kCols) : "memory");
}

// Few rows (decoding): one warp per output column, the weight row is read once with 16-byte loads and meets up to GV_ROWS
// activation rows; W streams from HBM at the copy rate, the activations come out of L1/L2.
constexpr int GV_ROWS = 8;
template <typename T> struct Vec8;
template <> struct Vec8<bf16> {
    static constexpr int N = 8;
    __device__ static void load(const bf16* p, float* o) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <> struct Vec8<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* o) {
        const float4 u = *reinterpret_cast<const float4*>(p);
        o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w;
    }
};
#include "lp_rows_tail.cuh"

template <typename T, int EPI>
__global__ void __launch_bounds__(256) lp_gemv_kernel(const T* __restrict__ X, int ldx, const T* __restrict__ W, int ldw, void* __restrict__ Y,
                                                      int ldy, int R, int N, int K, float alpha, int vec_ok, int stage, RowsTail tail, int nh,
                                                      ZStride zs, const float* __restrict__ bias) {
    // nh > 0: the N outputs are heads of nh columns; head z = n / nh reads X `zs.x` elements on and writes column z * zs.y + n % nh
    extern __shared__ __align__(16) uint8_t gv_smem[];
    const T* X0 = X;
    const int lane = threadIdx.x & 31;
    constexpr int VN = Vec8<T>::N;
    if (stage) {   // the activation rows once per block into shared memory (every warp of the block reads all of them)
        T* xs = reinterpret_cast<T*>(gv_smem);
        const int per_row = K / VN;
        for (int i = threadIdx.x; i < R * per_row; i += blockDim.x) {
            const int r = i / per_row, c = i - r * per_row;
            *reinterpret_cast<uint4*>(xs + (size_t)r * K + c * VN) = *reinterpret_cast<const uint4*>(X + (size_t)r * ldx + c * VN);
        }
        __syncthreads();
        X = xs;
        ldx = K;
    }
    for (int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); n < N; n += gridDim.x * (blockDim.x >> 5)) {
    const T* wr = W + (size_t)n * ldw;
    size_t ycol = n;
    if (nh > 0) {
        const int z = n / nh;
        X = X0 + (size_t)z * zs.x;
        ycol = (size_t)z * zs.y + (size_t)(n - z * nh);
    }
    for (int rb = 0; rb < R; rb += GV_ROWS) {
        const int nr = min(GV_ROWS, R - rb);
        float acc[GV_ROWS] = {};
        if (vec_ok) {
#pragma unroll 4
            for (int k = lane * VN; k < K; k += 32 * VN) {
                float wv[VN], xv[VN];
                Vec8<T>::load(wr + k, wv);
#pragma unroll
                for (int i = 0; i < GV_ROWS; i++) {
                    if (i < nr) {
                        Vec8<T>::load(X + (size_t)(rb + i) * ldx + k, xv);
#pragma unroll
                        for (int e = 0; e < VN; e++) acc[i] = fmaf(wv[e], xv[e], acc[i]);
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float wv = to_f(wr[k]);
#pragma unroll
                for (int i = 0; i < GV_ROWS; i++)
                    if (i < nr) acc[i] = fmaf(wv, to_f(X[(size_t)(rb + i) * ldx + k]), acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < GV_ROWS; i++) {
            if (i < nr) {
                const float s = wsum(acc[i]);
                if (lane == 0) epi_store<T, EPI>(Y, (size_t)(rb + i) * ldy + ycol, alpha * s + (bias ? bias[n] : 0.0f));
            }
        }
    }
    }
    if (tail.on) rows_tail<T>(tail);
}

// The same for a normed input: the block first norms the (few) rows of the f32 residual stream into shared memory -- rms over the
// row, times the norm weight, rounded to the compute type exactly as lp_rmsnorm_kernel does -- and then multiplies from there.
// Every block repeats the norm (the rows are a few KB out of L2); a launch and a round trip through global memory go away.
template <typename T, int EPI>
__global__ void __launch_bounds__(256) lp_gemv_norm_kernel(const float* __restrict__ X, const int* __restrict__ gather, const float* __restrict__ nw,
                                                           float eps, const T* __restrict__ W, void* __restrict__ Y, int ldy, int R, int N, int K,
                                                           float alpha, int center, T* __restrict__ hn_out) {
    extern __shared__ __align__(16) uint8_t gn_smem[];
    T* xs = reinterpret_cast<T*>(gn_smem);            // [R][K]
    __shared__ float red[8];
    __shared__ float inv_s, mean_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = 0; r < R; r++) {
        const float* xr = X + (size_t)(gather ? gather[r] : r) * K;
        float mean = 0.0f;
        if (center) {   // layer norm: the mean first
            float t = 0.0f;
            for (int k = threadIdx.x; k < K; k += 256) t += xr[k];
            t = wsum(t);
            if (lane == 0) red[warp] = t;
            __syncthreads();
            if (threadIdx.x == 0) {
                float u = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) u += red[i];
                mean_s = u / (float)K;
            }
            __syncthreads();
            mean = mean_s;
        }
        float ss = 0.0f;
        for (int k = threadIdx.x; k < K; k += 256) ss += (xr[k] - mean) * (xr[k] - mean);
        ss = wsum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) t += red[i];
            inv_s = 1.0f / sqrtf(t / (float)K + eps);
        }
        __syncthreads();
        const float inv = inv_s;
        for (int k = threadIdx.x; k < K; k += 256) {
            const T v = from_f<T>((xr[k] - mean) * inv * nw[k]);
            xs[(size_t)r * K + k] = v;
            if (hn_out && blockIdx.x == 0) hn_out[(size_t)r * K + k] = v;   // (a later kernel of the layer reads the normed rows too)
        }
    }
    __syncthreads();
    constexpr int VN = Vec8<T>::N;
    for (int n = blockIdx.x * 8 + warp; n < N; n += gridDim.x * 8) {
    const T* wr = W + (size_t)n * K;
    for (int rb = 0; rb < R; rb += GV_ROWS) {
        const int nr = min(GV_ROWS, R - rb);
        float acc[GV_ROWS] = {};
#pragma unroll 4
        for (int k = lane * VN; k < K; k += 32 * VN) {   // (K is a multiple of VN: checked by the host)
            float wv[VN], xv[VN];
            Vec8<T>::load(wr + k, wv);
#pragma unroll
            for (int i = 0; i < GV_ROWS; i++) {
                if (i < nr) {
                    Vec8<T>::load(xs + (size_t)(rb + i) * K + k, xv);
#pragma unroll
                    for (int e = 0; e < VN; e++) acc[i] = fmaf(wv[e], xv[e], acc[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < GV_ROWS; i++) {
            if (i < nr) {
                const float sum = wsum(acc[i]);
                if (lane == 0) epi_store<T, EPI>(Y, (size_t)(rb + i) * ldy + n, alpha * sum);
            }
        }
    }
    }
}

// ------------------------------------------------------------------------------------------------ windowed attention
// After the fused projection P[r] = [q | k | v | gate | ...]: per-head RMS norm of q and k (shared weight of size dim), q to qbuf,
// k and v to the run's cache rows at the row's position.  Cache of a run: K [cap][G * dim] then V [cap][G * vdim], f32.
struct AttnGeom {
    int H, G, dim, vdim, window, keep_first, qk_norm, out_gate;
    float scale, eps;
    int q_off, k_off, v_off, g_off;   // columns of P
    size_t kv_off;                    // byte offset of this layer run inside a slot's cache block
    int out_ld;                       // row pitch of the output (the two branches of a mixer share one buffer: [attention | memory])
    float out_scale;                  // weight of the branch in the mixer's sum, applied before the rounding to the compute type
    int fused_prep;                   // the attention kernel norms q / k and writes the row's K, V itself (decoding: no prep launch)
    int cap;                          // positions a slot's cache holds
    // options of the general softmax mixer (all off for the window-and-memory mixer)
    int chunk;                        // 1: the mask is chunks of `window` positions counted from position 0 instead of a sliding window
    float softcap;                    // > 0: score <- softcap tanh(score / softcap)
    float slope_exp;                  // > 0: score -= 2^(-slope_exp (h + 1) / H) (i - j)
    int v_in_k;                       // 1: there are no value rows; a value is the first vdim entries of its (single, G = 1) key row
    int sink_mode;                    // B200_SINK_*: one more term exp(c) in the softmax's denominator, without key or value
    const float* sink;                // [H]: c per head (B200_SINK_LEARNED)
    const float* vrot;                // [rows][vdim]: cos | sin of the angles that turn a row's summed values back, or null
};
// the extra term of the denominator as the start of the running (maximum, sum): a key with score c and no value
__device__ __forceinline__ bool attn_sink(const AttnGeom& a, int h, float* c) {
    if (a.sink_mode == B200_SINK_NONE) return false;
    *c = a.sink_mode == B200_SINK_LEARNED ? a.sink[h] : 0.0f;
    return true;
}
// pair (2m, 2m + 1) of a head's summed values turned by minus the row's angle: tab = cos [vdim / 2] | sin [vdim / 2]
__device__ __forceinline__ void attn_turn_back(const float* tab, int half, int m, float& u, float& v) {
    const float c = tab[m], s = tab[half + m];
    const float nu = u * c + v * s, nv = v * c - u * s;
    u = nu;
    v = nv;
}
// out_gate: 0 none, 1 = sigmoid of a gate column per value channel, 2 = one gate column per head
__device__ __forceinline__ float attn_gate(const AttnGeom& a, const float* gate_row, int h, int ch) {
    return a.out_gate == 1 ? sigmoid_f(gate_row[h * a.vdim + ch]) : a.out_gate == 2 ? sigmoid_f(gate_row[h]) : 1.0f;
}
// first visible key of position i outside the kept first tokens
__device__ __forceinline__ int attn_lo(const AttnGeom& a, int i) { return a.chunk ? (i / a.window) * a.window : max(0, i - a.window + 1); }
__device__ __forceinline__ float attn_slope(const AttnGeom& a, int h) { return a.slope_exp > 0.0f ? exp2f(-a.slope_exp * (float)(h + 1) / (float)a.H) : 0.0f; }
// what happens to a scaled score before the softmax
__device__ __forceinline__ float attn_score(const AttnGeom& a, float s, float slope, int i, int j) {
    if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
    return s - slope * (float)(i - j);
}
__global__ void lp_attn_prep_kernel(StepMeta sm, AttnGeom a, const float* __restrict__ P, int ldp, const float* __restrict__ qw,
                                    const float* __restrict__ kw, float* __restrict__ qbuf) {
    const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int run = sm.row_run[r], pos = sm.row_pos[r];
    const float* p = P + (size_t)r * ldp;
    float* kc = reinterpret_cast<float*>(sm.run_kv[run] + a.kv_off) + (size_t)pos * a.G * a.dim;
    float* vc = reinterpret_cast<float*>(sm.run_kv[run] + a.kv_off) + (size_t)a.cap * a.G * a.dim + (size_t)pos * a.G * a.vdim;
    for (int h = warp; h < a.H + a.G; h += nw) {
        const bool isq = h < a.H;
        const float* src = isq ? p + a.q_off + h * a.dim : p + a.k_off + (h - a.H) * a.dim;
        float* dst = isq ? qbuf + (size_t)r * a.H * a.dim + h * a.dim : kc + (h - a.H) * a.dim;
        const float* w = isq ? qw : kw;
        float inv = 1.0f;
        if (a.qk_norm) {
            float ss = 0.0f;
            for (int d = lane; d < a.dim; d += 32) ss += src[d] * src[d];
            ss = wsum(ss);
            inv = 1.0f / sqrtf(ss / (float)a.dim + a.eps);
        }
        for (int d = lane; d < a.dim; d += 32) dst[d] = a.qk_norm ? src[d] * inv * w[d] : src[d];
    }
    for (int c = threadIdx.x; c < a.G * a.vdim; c += blockDim.x) vc[c] = p[a.v_off + c];
}

// One block of ATT_WARPS warps per (row, query head).  Keys go in blocks of 32, dealt to the warps in turn: one key per lane for the
// scores (q from shared memory), online softmax in f32 per warp, then the block's 32 value rows are added lane-per-channel; the
// warps' partial (max, sum, output) triples are merged through shared memory.  Visible keys of position i: [0, min(keep_first, lo))
// and [lo, i], lo = max(0, i - window + 1).  The output is multiplied by sigmoid(gate) when the layer has an output gate.
constexpr int ATT_ACC = 16;   // value channels per lane at most: vdim <= 512 (the kernel is instantiated for 4, 8 and 16)
constexpr int ATT_WARPS = 16;
constexpr int ATT_QCH = 2;    // 16-byte query chunks per lane in the split-channel score loop: dim <= 256 (wider: one key per lane)
template <typename OutT, int VCH>
__global__ void __launch_bounds__(32 * ATT_WARPS) lp_window_attn_kernel(StepMeta sm, AttnGeom a, const float* __restrict__ qbuf,
                                                                        const float* __restrict__ P, int ldp, const float* __restrict__ qw,
                                                                        const float* __restrict__ kw, OutT* __restrict__ out) {
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                                  // [dim]
    float* acc_s = smem + ((a.dim + 3) & ~3);          // [ATT_WARPS][vdim]
    float* ml_s = acc_s + ATT_WARPS * a.vdim;          // [ATT_WARPS][2]
    float* om = ml_s + 2 * ATT_WARPS;                  // [vdim] (with vrot only)
    const int r = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int run = sm.row_run[r], i = sm.row_pos[r];
    const int g = h * a.G / a.H;
    const float* kc = reinterpret_cast<const float*>(sm.run_kv[run] + a.kv_off);
    const float* vc = a.v_in_k ? kc : kc + (size_t)a.cap * a.G * a.dim;
    const int ldk = a.G * a.dim, ldv = a.v_in_k ? ldk : a.G * a.vdim;
    if (a.fused_prep) {
        // what lp_attn_prep_kernel does, for this head and its K/V group only: warp 0 norms q into shared memory, warp 1 norms k
        // into the cache row of this position, the other warps copy v there.  Every head of a group writes the same values; a
        // block reads back its own writes after the barrier.
        const float* p = P + (size_t)r * ldp;
        if (warp < 2) {
            const float* src = warp ? p + a.k_off + g * a.dim : p + a.q_off + h * a.dim;
            float* dst = warp ? const_cast<float*>(kc) + (size_t)i * ldk + g * a.dim : qs;
            const float* w = warp ? kw : qw;
            float inv = 1.0f;
            if (a.qk_norm) {
                float ss = 0.0f;
                for (int d = lane; d < a.dim; d += 32) ss += src[d] * src[d];
                ss = wsum(ss);
                inv = 1.0f / sqrtf(ss / (float)a.dim + a.eps);
            }
            for (int d = lane; d < a.dim; d += 32) dst[d] = a.qk_norm ? src[d] * inv * w[d] : src[d];
        } else {
            float* dst = const_cast<float*>(vc) + (size_t)i * ldv + g * a.vdim;
            for (int c = threadIdx.x - 64; c < a.vdim; c += blockDim.x - 64) dst[c] = p[a.v_off + g * a.vdim + c];
        }
        __threadfence_block();
    } else {
        const float* q = qbuf + (size_t)r * a.H * a.dim + h * a.dim;
        for (int d = threadIdx.x; d < a.dim; d += blockDim.x) qs[d] = q[d];
    }
    __syncthreads();
    const int lo = attn_lo(a, i);
    const int a_end = min(a.keep_first, lo);
    const int nb0 = (a_end + 31) >> 5, nb1 = (i + 1 - lo + 31) >> 5;
    const float slope = attn_slope(a, h);
    float m = -INFINITY, l = 0.0f;
    {
        float c;
        if (warp == 0 && attn_sink(a, h, &c)) { m = c; l = 1.0f; }
    }
    float acc[VCH];
#pragma unroll
    for (int c = 0; c < VCH; c++) acc[c] = 0.0f;
    const bool v4 = (a.dim & 3) == 0 && a.dim <= 128 * ATT_QCH;
    float4 qr[ATT_QCH];
#pragma unroll
    for (int c = 0; c < ATT_QCH; c++) {
        const int d = (lane + 32 * c) * 4;
        qr[c] = (v4 && d < a.dim) ? *reinterpret_cast<const float4*>(qs + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int b = warp; b < nb0 + nb1; b += ATT_WARPS) {
        const int j0 = b < nb0 ? b * 32 : lo + (b - nb0) * 32;
        const int end = b < nb0 ? a_end : i + 1;
        const int j = j0 + lane;
        float s = -INFINITY;
        if (v4) {
            // lanes split the key channels (coalesced 16-byte loads of one cache row per key), a butterfly sums the partial dots
            const int cnt = min(32, end - j0);
            for (int jb = 0; jb < cnt; jb += 8) {      // eight keys at a time: all their loads first, then the eight butterflies
                float part[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    part[u] = 0.0f;
                    if (jb + u < cnt) {
                        const float* kr = kc + (size_t)(j0 + jb + u) * ldk + g * a.dim;
#pragma unroll
                        for (int c = 0; c < ATT_QCH; c++) {
                            const int d = (lane + 32 * c) * 4;
                            if (d < a.dim) {
                                const float4 kv = *reinterpret_cast<const float4*>(kr + d);
                                part[u] = fmaf(qr[c].x, kv.x, part[u]);
                                part[u] = fmaf(qr[c].y, kv.y, part[u]);
                                part[u] = fmaf(qr[c].z, kv.z, part[u]);
                                part[u] = fmaf(qr[c].w, kv.w, part[u]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float tot = wsum(part[u]);
                    if (lane == jb + u && jb + u < cnt) s = tot * a.scale;
                }
            }
        } else if (j < end) {
            const float* kr = kc + (size_t)j * ldk + g * a.dim;
            float d0 = 0.0f;
            for (int d = 0; d < a.dim; d++) d0 = fmaf(qs[d], kr[d], d0);
            s = d0 * a.scale;
        }
        if (j < end) s = attn_score(a, s, slope, i, j);
        const float m_new = fmaxf(m, wmax(s));
        const float p = j < end ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);      // (m = -inf on the warp's first block: 0)
        l = l * corr + wsum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < VCH; c++) acc[c] *= corr;
        const int cnt = min(32, end - j0);
        constexpr int PVB = VCH <= 4 ? 8 : 4;          // value rows per batch: weights first, then all loads, then the sums
        for (int jb = 0; jb < cnt; jb += PVB) {
            float pj[PVB];
#pragma unroll
            for (int u = 0; u < PVB; u++) pj[u] = __shfl_sync(0xffffffffu, p, (jb + u) & 31);
            float vv[PVB][VCH];
#pragma unroll
            for (int u = 0; u < PVB; u++) {
                const float* vr = vc + (size_t)(j0 + min(jb + u, cnt - 1)) * ldv + g * a.vdim;
#pragma unroll
                for (int c = 0; c < VCH; c++) {
                    const int ch = c * 32 + lane;
                    vv[u][c] = ch < a.vdim ? vr[ch] : 0.0f;
                }
                if (jb + u >= cnt) pj[u] = 0.0f;
            }
#pragma unroll
            for (int u = 0; u < PVB; u++)
#pragma unroll
                for (int c = 0; c < VCH; c++) acc[c] = fmaf(pj[u], vv[u][c], acc[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < VCH; c++) {
        const int ch = c * 32 + lane;
        if (ch < a.vdim) acc_s[warp * a.vdim + ch] = acc[c];
    }
    if (lane == 0) {
        ml_s[2 * warp] = m;
        ml_s[2 * warp + 1] = l;
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, ml_s[2 * w]);
    float wgt[ATT_WARPS], lsum = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) {
        wgt[w] = expf(ml_s[2 * w] - M);           // a warp without keys: exp(-inf) = 0
        lsum = fmaf(ml_s[2 * w + 1], wgt[w], lsum);
    }
    const float invl = 1.0f / lsum;
    const float* gate = P + (size_t)r * ldp + a.g_off;
    if (a.vrot) {   // the merged sums first, then every pair is turned back by the row's angle
        for (int ch = threadIdx.x; ch < a.vdim; ch += blockDim.x) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++) o = fmaf(acc_s[w * a.vdim + ch], wgt[w], o);
            om[ch] = o * invl;
        }
        __syncthreads();
        const float* tab = a.vrot + (size_t)r * a.vdim;
        for (int pm = threadIdx.x; pm < a.vdim / 2; pm += blockDim.x) {
            float u = om[2 * pm], v = om[2 * pm + 1];
            attn_turn_back(tab, a.vdim / 2, pm, u, v);
            out[(size_t)r * a.out_ld + h * a.vdim + 2 * pm] = from_f<OutT>(u * attn_gate(a, gate, h, 2 * pm) * a.out_scale);
            out[(size_t)r * a.out_ld + h * a.vdim + 2 * pm + 1] = from_f<OutT>(v * attn_gate(a, gate, h, 2 * pm + 1) * a.out_scale);
        }
        return;
    }
    for (int ch = threadIdx.x; ch < a.vdim; ch += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) o = fmaf(acc_s[w * a.vdim + ch], wgt[w], o);
        o *= invl;
        o *= attn_gate(a, gate, h, ch);
        out[(size_t)r * a.out_ld + h * a.vdim + ch] = from_f<OutT>(o * a.out_scale);
    }
}

// Prompt rows in bf16 mode: 64 queries of one (run, head) per block, 16 per warp, against key tiles of 64 staged in shared memory as
// bf16 (K as [key][dim], V transposed as [channel][key]); scores and the value sum run on the tensor pipe (mma.sync m16n8k16, bf16
// operands, f32 accumulators), the mask, the online softmax and the normalisation in f32 registers.  The probabilities go from
// the accumulator layout of the score tile straight into the A operand of the value product.  DK / DV are upper bounds of the key
// and value sizes (multiples of 16 / 8 at run time); the visible keys of a tile of queries are [0, min(keep_first, lo0)) and
// [lo0, last query], lo0 = the window start of its first query, every element masked by the rule itself.
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int AT_Q = 64, AT_K = 64;
template <int DK, int DV>
__global__ void __launch_bounds__(128) lp_window_attn_tile_kernel(StepMeta sm, AttnGeom a, const float* __restrict__ qbuf,
                                                                  const float* __restrict__ P, int ldp, bf16* __restrict__ out) {
    constexpr int KS = DK + 8, VS = AT_K + 8;          // row pitches in bf16: conflict-free 32-bit fragment loads
    extern __shared__ __align__(16) uint8_t at_smem[];
    bf16* Ks = reinterpret_cast<bf16*>(at_smem);        // [AT_K][KS]
    bf16* Vt = Ks + AT_K * KS;                          // [DV][VS]
    const int run = blockIdx.z, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int r0 = sm.run_start[run], len = sm.run_start[run + 1] - r0, p0 = sm.run_pos0[run];
    const int t0 = blockIdx.x * AT_Q;
    if (t0 >= len) return;
    const int g = h * a.G / a.H;
    const float* kc = reinterpret_cast<const float*>(sm.run_kv[run] + a.kv_off);
    const float* vc = a.v_in_k ? kc : kc + (size_t)a.cap * a.G * a.dim;
    const int ldk = a.G * a.dim, ldv = a.v_in_k ? ldk : a.G * a.vdim;
    // this thread's two query rows (gid and gid + 8 of the warp's 16) and their positions
    const int tq0 = t0 + warp * 16 + gid, tq1 = tq0 + 8;
    const int i0 = p0 + tq0, i1 = p0 + tq1;
    const bool ok0 = tq0 < len, ok1 = tq1 < len;
    uint32_t qa[DK / 16][4];
#pragma unroll
    for (int kb = 0; kb < DK / 16; kb++) {
        const int d = kb * 16 + 2 * tig;
        const float* q0 = qbuf + (size_t)(r0 + tq0) * a.H * a.dim + h * a.dim;
        const float* q1 = qbuf + (size_t)(r0 + tq1) * a.H * a.dim + h * a.dim;
        const bool in = d < a.dim;       // dim is a multiple of 16: d + 9 < dim too
        qa[kb][0] = (ok0 && in) ? pack_bf2(q0[d], q0[d + 1]) : 0u;
        qa[kb][1] = (ok1 && in) ? pack_bf2(q1[d], q1[d + 1]) : 0u;
        qa[kb][2] = (ok0 && in) ? pack_bf2(q0[d + 8], q0[d + 9]) : 0u;
        qa[kb][3] = (ok1 && in) ? pack_bf2(q1[d + 8], q1[d + 9]) : 0u;
    }
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    {
        float c;
        if (attn_sink(a, h, &c)) { m0 = m1 = c; l0 = l1 = 1.0f; }
    }
    const int first = p0 + t0, last = p0 + min(t0 + AT_Q, len) - 1;
    const int lo0 = attn_lo(a, first);
    const int a_end = min(a.keep_first, lo0);
    const float slope = attn_slope(a, h);
    for (int part = 0; part < 2; part++) {
        const int beg = part ? lo0 : 0, end = part ? last + 1 : a_end;
        for (int j0 = beg; j0 < end; j0 += AT_K) {
            const int nk = min(AT_K, end - j0);
            __syncthreads();   // the previous tile has been consumed
            // K: a thread takes 4 channels of one key per round (coalesced rows), all loads of a batch before their stores
            {
                constexpr int KN = AT_K * (DK / 4) / 128;          // 16-byte loads per thread
#pragma unroll
                for (int b0 = 0; b0 < KN; b0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = threadIdx.x + (b0 + u) * 128, key = i / (DK / 4), d = (i - key * (DK / 4)) * 4;
                        v[u] = (key < nk && d < a.dim) ? *reinterpret_cast<const float4*>(kc + (size_t)(j0 + key) * ldk + g * a.dim + d)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = threadIdx.x + (b0 + u) * 128, key = i / (DK / 4), d = (i - key * (DK / 4)) * 4;
                        uint2 w;
                        w.x = pack_bf2(v[u].x, v[u].y);
                        w.y = pack_bf2(v[u].z, v[u].w);
                        *reinterpret_cast<uint2*>(Ks + key * KS + d) = w;
                    }
                }
            }
            // V transposed: neighbouring lanes take neighbouring keys of the same 4 channels, so the 2-byte stores of a warp fall into
            // neighbouring words of a channel's row (the row-major reads of a key are spread over rounds and come out of L1)
            {
                constexpr int VN4 = AT_K * (DV / 4) / 128;
#pragma unroll
                for (int b0 = 0; b0 < VN4; b0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = threadIdx.x + (b0 + u) * 128, key = i % AT_K, c = (i / AT_K) * 4;
                        v[u] = (key < nk && c < a.vdim) ? *reinterpret_cast<const float4*>(vc + (size_t)(j0 + key) * ldv + g * a.vdim + c)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = threadIdx.x + (b0 + u) * 128, key = i % AT_K, c = (i / AT_K) * 4;
                        Vt[(c + 0) * VS + key] = __float2bfloat16_rn(v[u].x);
                        Vt[(c + 1) * VS + key] = __float2bfloat16_rn(v[u].y);
                        Vt[(c + 2) * VS + key] = __float2bfloat16_rn(v[u].z);
                        Vt[(c + 3) * VS + key] = __float2bfloat16_rn(v[u].w);
                    }
                }
            }
            __syncthreads();
            // scores of 16 queries x 64 keys
            float sc[AT_K / 8][4];
#pragma unroll
            for (int n = 0; n < AT_K / 8; n++) {
                sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
                const bf16* kr = Ks + (n * 8 + gid) * KS + 2 * tig;
#pragma unroll
                for (int kb = 0; kb < DK / 16; kb++) {
                    if (kb * 16 < a.dim) {
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + kb * 16);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + kb * 16 + 8);
                        mma_bf16(sc[n], qa[kb], b0, b1);
                    }
                }
            }
            // mask, scale, running maximum per row
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < AT_K / 8; n++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = n * 8 + 2 * tig + (e & 1), j = j0 + key;
                    const int i = (e & 2) ? i1 : i0;
                    const bool vis = key < nk && ((e & 2) ? ok1 : ok0) && j <= i &&
                                     (a.chunk ? i / a.window == j / a.window : (i - j < a.window || j < a.keep_first));
                    sc[n][e] = vis ? attn_score(a, sc[n][e] * a.scale, slope, i, j) : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            const float c0 = n0 == -INFINITY ? 1.0f : expf(m0 - n0), c1 = n1 == -INFINITY ? 1.0f : expf(m1 - n1);
            m0 = n0;
            m1 = n1;
            float s0 = 0.0f, s1 = 0.0f;
            uint32_t pa[AT_K / 16][4];
#pragma unroll
            for (int n = 0; n < AT_K / 8; n++) {
                const float e0 = n0 == -INFINITY ? 0.0f : expf(sc[n][0] - n0), e1 = n0 == -INFINITY ? 0.0f : expf(sc[n][1] - n0);
                const float e2 = n1 == -INFINITY ? 0.0f : expf(sc[n][2] - n1), e3 = n1 == -INFINITY ? 0.0f : expf(sc[n][3] - n1);
                s0 += e0 + e1;
                s1 += e2 + e3;
                pa[n >> 1][(n & 1) * 2] = pack_bf2(e0, e1);
                pa[n >> 1][(n & 1) * 2 + 1] = pack_bf2(e2, e3);
            }
            s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
            s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
            s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
            s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
            l0 = l0 * c0 + s0;
            l1 = l1 * c1 + s1;
#pragma unroll
            for (int n = 0; n < DV / 8; n++) {
                if (n * 8 < a.vdim) {
                    o[n][0] *= c0;
                    o[n][1] *= c0;
                    o[n][2] *= c1;
                    o[n][3] *= c1;
                    const bf16* vr = Vt + (n * 8 + gid) * VS + 2 * tig;
#pragma unroll
                    for (int kb = 0; kb < AT_K / 16; kb++) {
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(vr + kb * 16);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(vr + kb * 16 + 8);
                        mma_bf16(o[n], pa[kb], b0, b1);
                    }
                }
            }
        }
    }
    const float inv0 = ok0 ? a.out_scale / l0 : 0.0f, inv1 = ok1 ? a.out_scale / l1 : 0.0f;
    const float* gate0 = P + (size_t)(r0 + tq0) * ldp + a.g_off;
    const float* gate1 = P + (size_t)(r0 + tq1) * ldp + a.g_off;
    bf16* out0 = out + (size_t)(r0 + tq0) * a.out_ld + h * a.vdim;
    bf16* out1 = out + (size_t)(r0 + tq1) * a.out_ld + h * a.vdim;
#pragma unroll
    for (int n = 0; n < DV / 8; n++) {
        const int ch = n * 8 + 2 * tig;
        if (ch < a.vdim) {
            if (ok0) {
                const float g0 = attn_gate(a, gate0, h, ch), g1 = attn_gate(a, gate0, h, ch + 1);
                float u = o[n][0] * inv0, v = o[n][1] * inv0;
                if (a.vrot) attn_turn_back(a.vrot + (size_t)(r0 + tq0) * a.vdim, a.vdim / 2, ch >> 1, u, v);
                *reinterpret_cast<uint32_t*>(out0 + ch) = pack_bf2(u * g0, v * g1);
            }
            if (ok1) {
                const float g0 = attn_gate(a, gate1, h, ch), g1 = attn_gate(a, gate1, h, ch + 1);
                float u = o[n][2] * inv1, v = o[n][3] * inv1;
                if (a.vrot) attn_turn_back(a.vrot + (size_t)(r0 + tq1) * a.vdim, a.vdim / 2, ch >> 1, u, v);
                *reinterpret_cast<uint32_t*>(out1 + ch) = pack_bf2(u * g0, v * g1);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ matrix memory
// Per (run, head): S [dim][vdim], n [dim], m; thread = value channel j, its column S[:, j] lives in registers for the whole run.
//   i = cap tanh((zi + bi) / cap),  f = logsigmoid(cap tanh((zf + bf) / cap)),  m' = max(f + m, i)
//   S <- e^(f + m - m') S + e^(i - m') k v^T,  n likewise with k,  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),  q = (W_q h) dim^(-1/2)
// State block of a run: S [H][dim][vdim] | n [H][dim] | m [H], f32.
struct MemGeom {
    int H, dim, vdim;
    float cap;
    int q_off, k_off, v_off, i_off, f_off;
    size_t rec_off;
};
constexpr int SCAN_BD = 64, SCAN_DREG = 16;
// How the scans are laid out.  A state column S[:, j] is cut into pieces of SCAN_DREG = 16 key channels, one piece per thread in
// registers (groups of four channels dealt round robin, so that the lanes of a column read neighbouring 16-byte words of shared
// memory): DMAX / 16 neighbouring lanes share a column (partial dot products meet through shuffles) and a block of 64 threads covers
// 64 / (DMAX / 16) columns, so wide keys mean more blocks and a shorter serial chain per token, not more registers.  Tokens are staged
// SCAN_CH at a time with 4-byte cp.async copies (all in flight together: one global round trip per chunk), gates and unit norms are
// worked out one token per thread / warp, and the serial loop over the chunk's tokens runs out of shared memory and registers.
template <int DMAX> struct ScanChunk { static constexpr int N = DMAX > 128 ? 16 : 32; };
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
template <int SPLIT>
__device__ __forceinline__ float split_sum(float v) {   // sum over the SPLIT neighbouring lanes that share a column
#pragma unroll
    for (int o = 1; o < SPLIT; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <int DMAX>
__global__ void __launch_bounds__(SCAN_BD) lp_matrix_memory_kernel(StepMeta sm, MemGeom g, const float* __restrict__ P, int ldp,
                                                                   const float* __restrict__ ib, const float* __restrict__ fb,
                                                                   float* __restrict__ O, int ldo) {
    constexpr int CH = ScanChunk<DMAX>::N, SPLIT = DMAX / SCAN_DREG, COLS = SCAN_BD / SPLIT;
    __shared__ __align__(16) float qs[CH][DMAX];
    __shared__ __align__(16) float ks[CH][DMAX];
    __shared__ float vs[CH][COLS], il_s[CH], fl_s[CH];
    const int tid = threadIdx.x, lane = tid & 31, col = tid / SPLIT, sub = tid % SPLIT;
    const int j = blockIdx.x * COLS + col, h = blockIdx.y, run = blockIdx.z;
    const int r0 = sm.run_start[run], r1 = sm.run_start[run + 1];
    float* Sg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)h * g.dim * g.vdim;
    float* ng = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)g.H * g.dim * g.vdim + (size_t)h * g.dim;
    float* mg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)g.H * g.dim * g.vdim + (size_t)g.H * g.dim + h;
    const bool live = j < g.vdim;
    float s[SCAN_DREG];
#pragma unroll
    for (int i = 0; i < SCAN_DREG; i++) {
        const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);   // channel of register i
        s[i] = (live && d < g.dim) ? Sg[(size_t)d * g.vdim + j] : 0.0f;
    }
    float nreg[DMAX / 32];   // n, element lane + 32 i (every warp keeps its own copy)
#pragma unroll
    for (int i = 0; i < DMAX / 32; i++) nreg[i] = lane + 32 * i < g.dim ? ng[lane + 32 * i] : 0.0f;
    for (int i = tid; i < CH * DMAX; i += SCAN_BD) {   // the padding beyond dim stays zero
        (&qs[0][0])[i] = 0.0f;
        (&ks[0][0])[i] = 0.0f;
    }
    float m = *mg;
    const float qscale = 1.0f / sqrtf((float)g.dim);
    const float bi = ib[h], bf_ = fb[h];
    const int jc = blockIdx.x * COLS + (tid % COLS);   // the column this thread stages
    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();   // the previous chunk has been consumed
        for (int t = 0; t < nt; t++) {
            const float* p = P + (size_t)(c0 + t) * ldp;
            for (int d = tid; d < g.dim; d += SCAN_BD) {
                cp_async4(&qs[t][d], p + g.q_off + h * g.dim + d);
                cp_async4(&ks[t][d], p + g.k_off + h * g.dim + d);
            }
        }
        for (int t = tid / COLS; t < nt; t += SPLIT) {
            if (jc < g.vdim) cp_async4(&vs[t][tid % COLS], P + (size_t)(c0 + t) * ldp + g.v_off + h * g.vdim + jc);
            else vs[t][tid % COLS] = 0.0f;
        }
        if (tid < nt) {
            const float* p = P + (size_t)(c0 + tid) * ldp;
            il_s[tid] = g.cap * tanhf((p[g.i_off + h] + bi) / g.cap);
            fl_s[tid] = logsigmoid_f(g.cap * tanhf((p[g.f_off + h] + bf_) / g.cap));
        }
        cp_async_wait_all();
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float il = il_s[t], fl = fl_s[t];
            const float m_new = fmaxf(fl + m, il);
            const float fa = expf(fl + m - m_new), ia = expf(il - m_new);
            m = m_new;
            const float iv = ia * vs[t][col];
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_DREG; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][((i >> 2) * SPLIT + sub) * 4]);
                const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][((i >> 2) * SPLIT + sub) * 4]);
                s[i] = fmaf(fa, s[i], k4.x * iv);
                s[i + 1] = fmaf(fa, s[i + 1], k4.y * iv);
                s[i + 2] = fmaf(fa, s[i + 2], k4.z * iv);
                s[i + 3] = fmaf(fa, s[i + 3], k4.w * iv);
                a0 = fmaf(s[i], q4.x, a0);
                a1 = fmaf(s[i + 1], q4.y, a1);
                a2 = fmaf(s[i + 2], q4.z, a2);
                a3 = fmaf(s[i + 3], q4.w, a3);
            }
            float nq = 0.0f;
#pragma unroll
            for (int i = 0; i < DMAX / 32; i++) {
                nreg[i] = fmaf(fa, nreg[i], ia * ks[t][lane + 32 * i]);
                nq = fmaf(nreg[i], qs[t][lane + 32 * i], nq);
            }
            nq = wsum(nq) * qscale;
            const float acc = split_sum<SPLIT>((a0 + a1) + (a2 + a3)) * qscale;
            if (live && sub == 0) O[(size_t)(c0 + t) * ldo + h * g.vdim + j] = acc / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
        }
    }
    if (live)
#pragma unroll
        for (int i = 0; i < SCAN_DREG; i++) {
            const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);
            if (d < g.dim) Sg[(size_t)d * g.vdim + j] = s[i];
        }
    if (blockIdx.x == 0 && tid < 32) {
#pragma unroll
        for (int i = 0; i < DMAX / 32; i++)
            if (lane + 32 * i < g.dim) ng[lane + 32 * i] = nreg[i];
        if (tid == 0) *mg = m;
    }
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// Causal depthwise convolution + SiLU over the first C columns of P (q | k | v of the fused projection).  Weights [C][taps], the last
// tap meets the current token; inputs before a run's first row come from the run's tail (the last taps - 1 inputs, zero at the
// start of a sequence).  State block of a run: S [H][dim][vdim] | tail [taps - 1][C], f32.
struct DeltaGeom {
    int H, G, dim, vdim, taps, C;     // C = 2 G dim + H vdim; the state-space mixer borrows H, dim (= state), vdim, taps, C, in_off, rec_off
    int g_off, b_off, a_off;          // columns of P: gate | write strength | decay
    size_t rec_off;
    float eps;
    int in_off;                       // first convolved column of P
};
// (the convolved channels are columns in_off .. in_off + C of P; bias: one value per channel added to the sum, or null)
__global__ void lp_conv_silu_kernel(StepMeta sm, DeltaGeom g, const float* __restrict__ P, int ldp, const float* __restrict__ cw,
                                    const float* __restrict__ bias, float* __restrict__ out, int shift_tail) {
    const int r = blockIdx.x, run = sm.row_run[r];
    const int t = r - sm.run_start[run];
    float* tail = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)g.H * g.dim * g.vdim;
    P += g.in_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < g.C; c += gridDim.y * blockDim.x) {   // (channels are independent)
        float y = bias ? bias[c] : 0.0f;
        for (int i = 0; i < g.taps; i++) {
            const int tt = t - (g.taps - 1) + i;
            const float in = tt >= 0 ? P[(size_t)(r - t + tt) * ldp + c] : tail[(size_t)(g.taps - 1 + tt) * g.C + c];
            y = fmaf(cw[(size_t)c * g.taps + i], in, y);
        }
        out[(size_t)r * g.C + c] = y * sigmoid_f(y);
        if (shift_tail) {   // every run has one row (decoding): the tail moves on by this input, channel by channel
            for (int i = 0; i + 1 < g.taps - 1; i++) tail[(size_t)i * g.C + c] = tail[(size_t)(i + 1) * g.C + c];
            if (g.taps > 1) tail[(size_t)(g.taps - 2) * g.C + c] = P[(size_t)r * ldp + c];
        }
    }
}
// After the convolution: the run's tail becomes the last taps - 1 inputs of (old tail ++ new rows).
__global__ void lp_conv_tail_kernel(StepMeta sm, DeltaGeom g, const float* __restrict__ P, int ldp) {
    const int run = blockIdx.x, r0 = sm.run_start[run], len = sm.run_start[run + 1] - r0;
    float* tail = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)g.H * g.dim * g.vdim;
    P += g.in_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < g.C; c += gridDim.y * blockDim.x)
        for (int i = 0; i < g.taps - 1; i++) {
            const int st = len + i - (g.taps - 1);
            tail[(size_t)i * g.C + c] = st >= 0 ? P[(size_t)(r0 + st) * ldp + c] : tail[(size_t)(i + len) * g.C + c];
        }
}
// Per (run, head), laid out like the matrix-memory scan.  q, k become unit vectors (x / sqrt(sum x^2 + 1e-6), q also times
// dim^(-1/2)): a warp normalises one staged vector at a time in shared memory; beta = sigmoid(zb);
// decay = exp(-exp(A_log) softplus(za + dt_bias));
//   S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (the read-out sees this token's write).
template <int DMAX>
__global__ void __launch_bounds__(SCAN_BD) lp_gated_delta_kernel(StepMeta sm, DeltaGeom g, const float* __restrict__ QKV, const float* __restrict__ P,
                                                                 int ldp, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                                 float* __restrict__ O, int ldo) {
    constexpr int CH = ScanChunk<DMAX>::N, SPLIT = DMAX / SCAN_DREG, COLS = SCAN_BD / SPLIT;
    __shared__ __align__(16) float qs[CH][DMAX];
    __shared__ __align__(16) float ks[CH][DMAX];
    __shared__ float vs[CH][COLS], beta_s[CH], dec_s[CH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, col = tid / SPLIT, sub = tid % SPLIT;
    const int j = blockIdx.x * COLS + col, h = blockIdx.y, run = blockIdx.z;
    const int hk = h * g.G / g.H;
    const int r0 = sm.run_start[run], r1 = sm.run_start[run + 1];
    float* Sg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)h * g.dim * g.vdim;
    const bool live = j < g.vdim;
    float s[SCAN_DREG];
#pragma unroll
    for (int i = 0; i < SCAN_DREG; i++) {
        const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);   // channel of register i
        s[i] = (live && d < g.dim) ? Sg[(size_t)d * g.vdim + j] : 0.0f;
    }
    for (int i = tid; i < CH * DMAX; i += SCAN_BD) {
        (&qs[0][0])[i] = 0.0f;
        (&ks[0][0])[i] = 0.0f;
    }
    const float rate = expf(A_log[h]), dtb = dt_bias[h];
    const float qscale = 1.0f / sqrtf((float)g.dim);
    const int k_col = g.G * g.dim, v_col = 2 * g.G * g.dim;
    const int jc = blockIdx.x * COLS + (tid % COLS);
    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float* x = QKV + (size_t)(c0 + t) * g.C + hk * g.dim;
            for (int d = tid; d < g.dim; d += SCAN_BD) {
                cp_async4(&qs[t][d], x + d);
                cp_async4(&ks[t][d], x + k_col + d);
            }
        }
        for (int t = tid / COLS; t < nt; t += SPLIT) {
            if (jc < g.vdim) cp_async4(&vs[t][tid % COLS], QKV + (size_t)(c0 + t) * g.C + v_col + h * g.vdim + jc);
            else vs[t][tid % COLS] = 0.0f;
        }
        if (tid < nt) {
            const float* p = P + (size_t)(c0 + tid) * ldp;
            beta_s[tid] = sigmoid_f(p[g.b_off + h]);
            dec_s[tid] = expf(-rate * softplus_f(p[g.a_off + h] + dtb));
        }
        cp_async_wait_all();
        __syncthreads();
        for (int t = warp; t < 2 * nt; t += SCAN_BD / 32) {   // (token, q or k) pairs, one per warp at a time
            float* vec = (t & 1) ? ks[t >> 1] : qs[t >> 1];
            float ss = 0.0f;
            for (int d = lane; d < g.dim; d += 32) ss += vec[d] * vec[d];
            ss = wsum(ss);
            const float inv = ((t & 1) ? 1.0f : qscale) / sqrtf(ss + 1e-6f);
            for (int d = lane; d < g.dim; d += 32) vec[d] *= inv;
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float decay = dec_s[t], beta = beta_s[t], v = vs[t][col];
            float k0 = 0.0f, k1 = 0.0f, k2 = 0.0f, k3 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_DREG; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][((i >> 2) * SPLIT + sub) * 4]);
                s[i] *= decay;
                s[i + 1] *= decay;
                s[i + 2] *= decay;
                s[i + 3] *= decay;
                k0 = fmaf(s[i], k4.x, k0);
                k1 = fmaf(s[i + 1], k4.y, k1);
                k2 = fmaf(s[i + 2], k4.z, k2);
                k3 = fmaf(s[i + 3], k4.w, k3);
            }
            const float u = beta * (v - split_sum<SPLIT>((k0 + k1) + (k2 + k3)));
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_DREG; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][((i >> 2) * SPLIT + sub) * 4]);
                const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][((i >> 2) * SPLIT + sub) * 4]);
                s[i] = fmaf(k4.x, u, s[i]);
                s[i + 1] = fmaf(k4.y, u, s[i + 1]);
                s[i + 2] = fmaf(k4.z, u, s[i + 2]);
                s[i + 3] = fmaf(k4.w, u, s[i + 3]);
                a0 = fmaf(s[i], q4.x, a0);
                a1 = fmaf(s[i + 1], q4.y, a1);
                a2 = fmaf(s[i + 2], q4.z, a2);
                a3 = fmaf(s[i + 3], q4.w, a3);
            }
            const float acc = split_sum<SPLIT>((a0 + a1) + (a2 + a3));
            if (live && sub == 0) O[(size_t)(c0 + t) * ldo + h * g.vdim + j] = acc;
        }
    }
    if (live)
#pragma unroll
        for (int i = 0; i < SCAN_DREG; i++) {
            const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);
            if (d < g.dim) Sg[(size_t)d * g.vdim + j] = s[i];
        }
}

// out[r][h][c] = o / sqrt(mean_c o^2 + eps) * w[w_per_head ? c : h * vdim + c] * act(gate), act = sigmoid (0), SiLU (1) or no gate at
// all (2); one warp per (row, head).  The result is the input of the mixer's output projection.
template <typename OutT>
__global__ void lp_headnorm_gate_kernel(const float* __restrict__ O, int ldo, const float* __restrict__ P, int ldp, int g_off,
                                        const float* __restrict__ w, int w_per_head, int H, int vdim, float eps, int act,
                                        OutT* __restrict__ out, int out_ld, float out_scale, int R) {
    const int r = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= H || r >= R) return;
    const float* o = O + (size_t)r * ldo + h * vdim;
    float ss = 0.0f;
    for (int c = lane; c < vdim; c += 32) ss += o[c] * o[c];
    ss = wsum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const float* gate = P + (size_t)r * ldp + g_off + h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        const float z = act == 2 ? 0.0f : gate[c];
        const float ga = act == 2 ? 1.0f : act ? z * sigmoid_f(z) : sigmoid_f(z);
        out[(size_t)r * out_ld + h * vdim + c] = from_f<OutT>(o[c] * inv * w[w_per_head ? c : h * vdim + c] * ga * out_scale);
    }
}

// Greedy pick per row, the LAST maximum wins (the rule of the library's other paths).
__global__ void lp_argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int bi = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (row[i] >= best) { best = row[i]; bi = i; }
    __shared__ float sv[1024];
    __shared__ int si[1024];
    sv[threadIdx.x] = best;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v2 = sv[threadIdx.x + o];
            const int i2 = si[threadIdx.x + o];
            if (v2 > sv[threadIdx.x] || (v2 == sv[threadIdx.x] && i2 > si[threadIdx.x])) { sv[threadIdx.x] = v2; si[threadIdx.x] = i2; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = si[0];
}

#include "lp_softmax_attn.cuh"
#include "lp_ffn.cuh"
#include "lp_streams.cuh"
#include "lp_latent_attn.cuh"
#include "lp_state_space.cuh"
#include "lp_gated_recurrent.cuh"

// out [H][b][a] = in [H][a][b]: a mixer's per-head matrices turned once at load
template <typename T>
__global__ void lp_transpose_heads_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int a, int b) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)H * a * b) return;
    const int h = (int)(i / ((size_t)a * b)), rem = (int)(i - (size_t)h * a * b), ia = rem / b, ib = rem - ia * b;
    out[(size_t)h * a * b + (size_t)ib * a + ia] = in[i];
}

__global__ void lp_add_scalar_kernel(float* __restrict__ v, int n, float a) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] += a;
}

// ------------------------------------------------------------------------------------------------ host side
struct Tensor {
    void* d = nullptr;      // matrices: compute type; vectors: f32
    bool matrix = false;
    uint64_t rows = 0, cols = 0;
    size_t bytes = 0;
};

struct LayerPlan {
    b200_layer_desc d{};
    // fused input projection of the mixer and its column map
    void* w_in = nullptr;
    int n_in = 0;
    AttnGeom ag{};
    MemGeom mg{};
    DeltaGeom dg{};
    const float *norm1 = nullptr, *norm2 = nullptr, *qn = nullptr, *kn = nullptr, *mem_norm = nullptr, *ib = nullptr, *fb = nullptr;
    const float *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr, *delta_norm = nullptr;
    void *wo_cat = nullptr, *wo_delta = nullptr, *w_up = nullptr, *w_down = nullptr;   // wo_cat: [width][attention | memory]
    int k_cat = 0;
    size_t kv_bytes = 0, rec_bytes = 0;   // per run, per slot (kv_bytes for `cap` positions)
    // general softmax mixer
    PrepGeom pg{};
    const float *qkv_bias = nullptr, *vmix = nullptr;
    const double* rot_freq = nullptr;
    void* wo = nullptr;
    // feed-forward: n_up rows of w_up ([up] | [gate | up] | [router | experts' up | always-on expert's up]), k_down columns of w_down
    int n_up = 0, k_down = 0;
    // latent attention: W_uq, W_uk turned per head ([H][kv_rank][dim]), W_uv ([H][vdim][kv_rank]); the run whose cache rows it reads
    LatentGeom lg{};
    void *w_uq = nullptr, *w_ukT = nullptr, *w_uv = nullptr;
    const float *dq_norm = nullptr, *dkv_norm = nullptr;
    float rot_mult = 1.0f;
    int kv_layer = -1;
    // state-space mixer
    SsdGeom sg{};
    const float *conv_b = nullptr, *ssd_D = nullptr, *ssd_norm = nullptr;
    // softmax mixer options: the extra term of the denominator per head, the output projection's bias, the values' own frequencies
    const float *sink = nullptr, *o_bias = nullptr;
    const double* v_freq = nullptr;
    // attention beside a recurrent unit: the unit's geometry and vectors, the right branch's own output projection and the two
    // branch norms (B200_COMBINE_NORMED_MEAN), the operand widths of the two branches
    GlinGeom gl{};
    GunitGeom gu{};
    const float *rec_b0 = nullptr, *rec_b1 = nullptr, *rec_lower = nullptr, *rec_norm = nullptr, *left_out = nullptr, *right_out = nullptr;
    void* wo_right = nullptr;
    int k_left = 0, k_right = 0;
    // parallel_ff: first column of the feed-forward's part ([gate | up], [up] or the router) in the layer's input projection
    int ff_off = -1;
    int up_router_rows = 0;      // rows of the router at the head of w_up (0 when the router sits in the layer's input projection)
    // multi-stream layer form: [in | out | mix] of the two sublayers (null: identity)
    const float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
};

struct SlotMem {
    uint8_t* kv = nullptr;
    uint8_t* rec = nullptr;
};

}  // namespace

struct LpModel {
    b200_program_desc p{};
    std::vector<b200_layer_desc> layers;
    int device = 0;
    cudaStream_t stream = nullptr;
    bool f32 = false, taps_on = false, finalized = false;
    std::map<std::string, Tensor> tensors;
    std::vector<LayerPlan> plan;        // per layer
    std::vector<int> runs;              // layer index of every layer run
    std::vector<int> run_pass;          // pass number t when the run is the first of a pass (step vector t is added), else -1
    std::vector<size_t> run_kv_off, run_rec_off;
    size_t slot_kv_bytes = 0, slot_rec_bytes = 0;
    std::vector<SlotMem> slot;          // per sequence slot; null = holds nothing
    std::vector<SlotMem> pool;
    double* inv_freq = nullptr;
    // per-step scratch (grow-only)
    int cap_rows = 0, cap_runs = 0, cap_want = 0;
    uint8_t* h_meta = nullptr;          // pinned
    uint8_t* d_meta = nullptr;
    size_t meta_bytes = 0;
    float *x = nullptr, *P = nullptr, *qbuf = nullptr, *O = nullptr, *conv = nullptr, *logits = nullptr;
    float *y = nullptr, *vsrc = nullptr, *moe_w = nullptr, *moe_selw = nullptr;   // sublayer output (norm-after-sum layers), shared values, routing
    float* xs = nullptr;                // [rows][streams][width]: the residual copies of the multi-stream layer form
    void* cq = nullptr;                 // [rows][max_qrank] compute type: the normed query latent
    int max_qrank = 0;
    int *moe_sel = nullptr, *moe_pos = nullptr, *moe_seg = nullptr;   // chosen experts per row; row of (token, choice) in expert order; {first, rows} per expert
    void* moe_xp = nullptr;             // the tokens' rows gathered in expert order, compute type
    float* moe_yp = nullptr;            // the experts' outputs in the same order
    int max_vsrc = 0, max_experts = 0, max_top = 0;
    float* vrot = nullptr;              // [rows][max_vrot]: cos | sin of the angles that turn a row's summed values back
    int max_vrot = 0;
    bool need_y2 = false;               // m->y holds two sublayer outputs per row (branches that are normed before they are summed)
    void *hn = nullptr, *act_a = nullptr, *hw = nullptr;
    int* pick = nullptr;
    float* h_logits = nullptr;          // pinned
    size_t h_logits_bytes = 0;
    int max_in = 0, max_act = 0, max_o = 0, max_conv = 0, max_q = 0;
    float* taps = nullptr;
    size_t taps_floats = 0;
    int taps_len = 0;
    std::string launch_fail;   // name and launch shape of the first kernel whose launch was refused since the last report
    uint64_t launches = 0, weight_bytes = 0, kv_bytes_per_pos = 0;
    // tensor-core GEMM: on for bf16 steps of at least tc_min_rows rows (B200_LP_TC=0 keeps the CUDA-core kernel); *tc_err is set by a
    // bounded wait that gave up
    bool use_tc = true;
    bool use_fuse = true;        // B200_LP_FUSE=0: every step of a layer as a kernel of its own (norm, projection, ...)
    bool use_attn_tile = true;   // B200_LP_ATTN_TILE=0: the warp kernel for prompts too
    bool use_glin_seg = true;    // B200_LP_GLIN_SEG=0: the gated linear memory always walks whole runs
    float* glin_carry = nullptr; // segment carries of the gated linear memory [runs][segments][heads][dim][vdim]
    size_t glin_carry_bytes = 0;
    bool use_stream_tail = true; // B200_LP_STREAM_TAIL=0: few rows of the multi-stream form launch lp_streams_kernel instead of the fused tails
    // decode steps replay a CUDA graph per (rows, wanted rows, head); a graph is void once a scratch buffer has moved (B200_LP_GRAPH=0: eager)
    struct Graph { cudaGraphExec_t exec = nullptr; uint64_t launches = 0, epoch = 0; bool warm = false; };
    std::map<uint64_t, Graph> graphs;
    uint64_t scratch_epoch = 1;
    bool use_graph = true;
    int tc_min_rows = 17;
    int* tc_err = nullptr;
    int* h_tc_err = nullptr;
    unsigned* tail_counter = nullptr;   // arrival counter of rows_tail (zero between kernels)
};

namespace {

int lp_fail(std::string* err, int code, const std::string& msg) {
    if (err) *err = msg;
    return code;
}
#define LCU(expr)                                                                                                     \
    do {                                                                                                              \
        cudaError_t e_ = (expr);                                                                                      \
        if (e_ != cudaSuccess) return lp_fail(err, B200_ERR_OPERATION_FAILED, std::string(#expr) + ": " + cudaGetErrorString(e_)); \
    } while (0)
#define LCU_ALLOC(expr)                                                                                                \
    do {                                                                                                               \
        cudaError_t e_ = (expr);                                                                                       \
        if (e_ != cudaSuccess) return lp_fail(err, B200_ERR_ALLOCATION_FAILED, std::string(#expr) + ": " + cudaGetErrorString(e_)); \
    } while (0)

size_t elt(const LpModel* m) { return m->f32 ? 4 : 2; }
size_t up16(size_t v) { return (v + 255) & ~(size_t)255; }

uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
}
float bf16_to_f32(uint16_t h) {
    const uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    int exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (!man) u = sign;
        else {
            exp = 127 - 15 + 1;
            while (!(man & 0x400u)) { man <<= 1; exp--; }
            u = sign | ((uint32_t)exp << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((uint32_t)(exp - 15 + 127) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

bool is_matrix_name(const std::string& n) {
    // everything a GEMM or the embedding gather reads; the rest (norm weights, biases, convolution taps, per-head constants, step
    // vectors) is kept in f32
    if (n == "embed" || n == "head") return true;
    static const char* suf[] = {".q", ".k", ".v", ".g", ".o", ".i", ".f", ".a", ".b", ".up", ".down", ".gate", ".router",
                                ".dq", ".uq", ".dkv", ".uk", ".uv", ".in", ".z", ".x"};
    for (const char* s : suf) {
        const size_t L = strlen(s);
        if (n.size() > L && n.compare(n.size() - L, L, s) == 0) return true;
    }
    return false;
}

const Tensor* find(const LpModel* m, const std::string& name) {
    auto it = m->tensors.find(name);
    return it == m->tensors.end() ? nullptr : &it->second;
}

template <typename... KArgs, typename... Args>
void launch(LpModel* m, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    kern<<<grid, block, smem, m->stream>>>(std::forward<Args>(args)...);
    m->launches++;
    if (m->launch_fail.empty()) {   // the first refused launch is remembered by name, so that the step's error says which kernel it was
        const cudaError_t e = cudaPeekAtLastError();
        if (e != cudaSuccess) {
            const char* name = nullptr;
            if (cudaFuncGetName(&name, (const void*)kern) != cudaSuccess || !name) name = "?";
            char buf[512];
            snprintf(buf, sizeof buf, "%s <<<(%u,%u,%u), (%u,%u,%u), %zu>>>: %s", name, grid.x, grid.y, grid.z, block.x, block.y, block.z, smem,
                     cudaGetErrorString(e));
            m->launch_fail = buf;
        }
    }
}

// The tensor-core GEMM takes bf16 operands whose rows are 16-byte aligned (K and the row pitches multiples of 8).
template <int TN>
bool tc_launch(LpModel* m, const bf16* x, int ldx, const bf16* w, int ldw, int N, int K, void* Y, int ldy, int R, float alpha, int epi, const int* seg,
               int groups, size_t wz, ZStride zs, const float* bias) {
    const size_t smem = (size_t)TC_STAGES * (TC_M + TN) * 128 + 1024;
    static bool once[EPI_COUNT][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto prep = [&](auto kern, int e) {
        if (dev >= 0 && dev < 64 && once[e][dev]) return true;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (dev >= 0 && dev < 64) once[e][dev] = true;
        return true;
    };
    dim3 grid((N + TC_M - 1) / TC_M, (R + TN - 1) / TN, groups), block(128);
#define LP_TC(E)                                                                                                                       \
    do {                                                                                                                               \
        if (!prep(lp_gemm_tc_kernel<TN, E>, E)) return false;                                                                          \
        launch(m, lp_gemm_tc_kernel<TN, E>, grid, block, smem, x, ldx, w, ldw, Y, ldy, R, N, K, alpha, m->tc_err, seg, wz, zs, bias);  \
    } while (0)
    if (epi == EPI_STORE) LP_TC(EPI_STORE);
    else if (epi == EPI_ADD) LP_TC(EPI_ADD);
    else if (epi == EPI_GELU) LP_TC(EPI_GELU);
    else LP_TC(EPI_RELU2);
#undef LP_TC
    return true;
}
bool tc_gemm(LpModel* m, const void* X, int ldx, const void* W, int ldw, int N, int K, void* Y, int ldy, int R, float alpha, int epi, const int* seg,
             int groups, size_t wz, ZStride zs, const float* bias) {
    if (m->f32 || !m->use_tc || R < m->tc_min_rows) return false;
    if (K % 8 || ldx % 8 || ldw % 8 || wz % 8 || zs.x % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return false;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (R <= 64) return tc_launch<64>(m, x, ldx, w, ldw, N, K, Y, ldy, R, alpha, epi, seg, groups, wz, zs, bias);
    if (R <= 128) return tc_launch<128>(m, x, ldx, w, ldw, N, K, Y, ldy, R, alpha, epi, seg, groups, wz, zs, bias);   // (wider token tiles move fewer operand bytes per FLOP: measured 2.5x on a 2048 x 8192 x 2048 product even at 128 CTAs)
    return tc_launch<256>(m, x, ldx, w, ldw, N, K, Y, ldy, R, alpha, epi, seg, groups, wz, zs, bias);
}

// Y = epi(alpha X W^T): rows of the step against a [N][K] matrix in the compute type.  Without `seg`, groups > 1 batches the product
// over heads: head z multiplies columns [z zs.x, z zs.x + K) of X with rows [z N, (z + 1) N) of W (wz = N ldw) into columns
// [z zs.y, z zs.y + N) of Y.
template <typename T>
void gemm_t(LpModel* m, const void* X, int ldx, const void* W, int ldw, int N, int K, void* Y, int ldy, int R, float alpha, int epi, const int* seg = nullptr,
            int groups = 1, size_t wz = 0, const RowsTail* tail = nullptr, ZStride zs = ZStride{0, 0}, const float* bias = nullptr) {
    const T* x = (const T*)X;
    const T* w = (const T*)W;
    if (R <= 2 * GV_ROWS && !seg) {
        constexpr int VN = Vec8<T>::N;
        const bool heads = groups > 1;
        const int vec_ok = (K % VN == 0 && ldx % VN == 0 && ldw % VN == 0 && zs.x % VN == 0 && ((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0) ? 1 : 0;
        // a few blocks per SM, each walking its share of the output columns with the activation rows staged once
        const int Nall = N * groups;
        dim3 grid(std::min((Nall + 7) / 8, 4 * 148)), block(256);
        const size_t xbytes = (size_t)R * K * sizeof(T);
        // (40 KB: the kernel's static shared memory counts against the 48 KB a launch gets without opting in)
        const int stage = (!heads && vec_ok && sizeof(T) * VN == 16 && xbytes <= 40 * 1024) ? 1 : 0;
        const size_t smem = stage ? xbytes : 0;
        const RowsTail tl = tail ? *tail : RowsTail{};
        const int nh = heads ? N : 0;
#define LP_GV(E) launch(m, lp_gemv_kernel<T, E>, grid, block, smem, x, ldx, w, ldw, Y, ldy, R, Nall, K, alpha, vec_ok, stage, tl, nh, zs, bias)
        if (epi == EPI_STORE) LP_GV(EPI_STORE);
        else if (epi == EPI_ADD) LP_GV(EPI_ADD);
        else if (epi == EPI_GELU) LP_GV(EPI_GELU);
        else LP_GV(EPI_RELU2);
#undef LP_GV
        return;
    }
    if (tc_gemm(m, X, ldx, W, ldw, N, K, Y, ldy, R, alpha, epi, seg, groups, wz, zs, bias)) return;
    dim3 grid((N + GB - 1) / GB, (R + GB - 1) / GB, groups), block(256);
#define LP_GM(E) launch(m, lp_gemm_kernel<T, E>, grid, block, 0, x, ldx, w, ldw, Y, ldy, R, N, K, alpha, seg, wz, zs, bias)
    if (epi == EPI_STORE) LP_GM(EPI_STORE);
    else if (epi == EPI_ADD) LP_GM(EPI_ADD);
    else if (epi == EPI_GELU) LP_GM(EPI_GELU);
    else LP_GM(EPI_RELU2);
#undef LP_GM
}
// tail: few rows only (the caller has checked R): the last block goes on with rows_tail
void gemm(LpModel* m, const void* X, int ldx, const void* W, int N, int K, void* Y, int ldy, int R, float alpha, int epi, const RowsTail* tail = nullptr,
          const float* bias = nullptr) {
    if (m->f32) gemm_t<float>(m, X, ldx, W, K, N, K, Y, ldy, R, alpha, epi, nullptr, 1, 0, tail, ZStride{0, 0}, bias);
    else gemm_t<bf16>(m, X, ldx, W, K, N, K, Y, ldy, R, alpha, epi, nullptr, 1, 0, tail, ZStride{0, 0}, bias);
}
// `groups` products in one launch (grid.z): group g multiplies rows [seg[2g], seg[2g] + seg[2g + 1]) of X -- the counts live on the
// device, R is their upper bound -- with the matrix at Wm + g * zs elements, whose rows are ldw apart (contiguous matrices: ldw = K,
// zs = N K; column blocks of one wide matrix: ldw = its width, zs = K), into the same rows of Y.
void gemm_grouped(LpModel* m, const void* X, int ldx, const void* Wm, int ldw, size_t zs, int groups, int N, int K, void* Y, int ldy, int R, int epi,
                  const int* seg) {
    if (m->f32) gemm_t<float>(m, X, ldx, Wm, ldw, N, K, Y, ldy, R, 1.0f, epi, seg, groups, zs);
    else gemm_t<bf16>(m, X, ldx, Wm, ldw, N, K, Y, ldy, R, 1.0f, epi, seg, groups, zs);
}
// One product per head in one launch: Y[r][z yz + n] = sum_k X[r][z xz + k] Wm[z N + n][k], z < heads, all rows of the step (f32 out).
void gemm_heads(LpModel* m, const void* X, int ldx, size_t xz, const void* Wm, int heads, int N, int K, void* Y, int ldy, size_t yz, int R) {
    if (m->f32) gemm_t<float>(m, X, ldx, Wm, K, N, K, Y, ldy, R, 1.0f, EPI_STORE, nullptr, heads, (size_t)N * K, nullptr, ZStride{xz, yz});
    else gemm_t<bf16>(m, X, ldx, Wm, K, N, K, Y, ldy, R, 1.0f, EPI_STORE, nullptr, heads, (size_t)N * K, nullptr, ZStride{xz, yz});
}
// One product with a weight matrix whose rows are `ldw` apart (a block of columns of a wider matrix).
void gemm_ld(LpModel* m, const void* X, int ldx, const void* Wm, int ldw, int N, int K, void* Y, int ldy, int R, int epi, const float* bias = nullptr) {
    if (m->f32) gemm_t<float>(m, X, ldx, Wm, ldw, N, K, Y, ldy, R, 1.0f, epi, nullptr, 1, 0, nullptr, ZStride{0, 0}, bias);
    else gemm_t<bf16>(m, X, ldx, Wm, ldw, N, K, Y, ldy, R, 1.0f, epi, nullptr, 1, 0, nullptr, ZStride{0, 0}, bias);
}

int norm_center(const LpModel* m) { return m->p.norm_kind == B200_NORM_LAYER ? 1 : 0; }

void rmsnorm(LpModel* m, float* x, const float* add, const float* w, void* out, const int* gather, int rows) {
    if (m->f32) launch(m, lp_rmsnorm_kernel<float>, dim3(rows), dim3(128), 0, x, add, w, (float*)out, gather, m->p.width, m->p.norm_eps, norm_center(m));
    else launch(m, lp_rmsnorm_kernel<bf16>, dim3(rows), dim3(128), 0, x, add, w, (bf16*)out, gather, m->p.width, m->p.norm_eps, norm_center(m));
}

// norm + projection of the step's rows: one fused kernel for a few rows (decoding) when the normed rows fit in shared memory,
// else lp_rmsnorm_kernel into `scratch` and a GEMM from there.  add: the pass vector of a repeated layer range (unfused: it is
// written back into the stream).
template <typename T>
bool gemv_norm_t(LpModel* m, const float* x, const int* gather, const float* nw, const void* W, int N, int K, void* Y, int ldy, int R, float alpha,
                 int epi, void* hn_out) {
    constexpr int VN = Vec8<T>::N;
    const size_t smem = (size_t)R * K * sizeof(T);
    if (R > 2 * GV_ROWS || K % VN || ((uintptr_t)W & 15) || smem > 96 * 1024) return false;
    static bool once[EPI_COUNT][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto prep = [&](auto kern, int e) {
        if (dev >= 0 && dev < 64 && once[e][dev]) return true;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (dev >= 0 && dev < 64) once[e][dev] = true;
        return true;
    };
    dim3 grid(std::min((N + 7) / 8, 4 * 148)), block(256);
    const T* w = (const T*)W;
    if (epi == EPI_STORE) {
        if (!prep(lp_gemv_norm_kernel<T, EPI_STORE>, 0)) return false;
        launch(m, lp_gemv_norm_kernel<T, EPI_STORE>, grid, block, smem, x, gather, nw, m->p.norm_eps, w, Y, ldy, R, N, K, alpha, norm_center(m), (T*)hn_out);
    } else if (epi == EPI_RELU2) {
        if (!prep(lp_gemv_norm_kernel<T, EPI_RELU2>, 2)) return false;
        launch(m, lp_gemv_norm_kernel<T, EPI_RELU2>, grid, block, smem, x, gather, nw, m->p.norm_eps, w, Y, ldy, R, N, K, alpha, norm_center(m), (T*)hn_out);
    } else return false;
    return true;
}
// keep: the normed rows are also wanted in `scratch` afterwards (the fused kernel then writes them out as well)
void norm_gemm(LpModel* m, float* x, const float* add, const int* gather, const float* nw, void* scratch, const void* W, int N, void* Y, int ldy,
               int R, float alpha, int epi, bool keep = false) {
    const int K = m->p.width;
    if (!add && m->use_fuse) {
        void* hn_out = keep ? scratch : nullptr;
        if (m->f32 ? gemv_norm_t<float>(m, x, gather, nw, W, N, K, Y, ldy, R, alpha, epi, hn_out) : gemv_norm_t<bf16>(m, x, gather, nw, W, N, K, Y, ldy, R, alpha, epi, hn_out))
            return;
    }
    rmsnorm(m, x, add, nw, scratch, gather, R);
    gemm(m, scratch, K, W, N, K, Y, ldy, R, alpha, epi);
}

int pick_dmax(int dim) { return dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256; }

}  // namespace

// ------------------------------------------------------------------------------------------------ create / upload / finalize
int lp_create(const b200_program_desc* prog, const b200_layer_desc* layers, int device, cudaStream_t stream, bool taps, LpModel** out,
              std::string* err) {
    if (!prog || !layers || !out) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_ctx_create_layers: null argument");
    const b200_program_desc& p = *prog;
    auto bad = [&](const std::string& s) { return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_ctx_create_layers: " + s); };
    if (p.width <= 0 || p.vocab <= 0 || p.n_layers <= 0 || p.max_seq_len <= 0 || p.max_batch <= 0) return bad("non-positive model dimension");
    if (p.compute != B200_COMPUTE_BF16 && p.compute != B200_COMPUTE_F32) return bad("compute must be B200_COMPUTE_BF16 or B200_COMPUTE_F32");
    const bool looped = p.loop_stop > p.loop_start;
    if (looped && (p.loop_start < 0 || p.loop_stop > p.n_layers || p.loop_times < 1)) return bad("bad repeated layer range");
    if (p.norm_kind != B200_NORM_RMS && p.norm_kind != B200_NORM_LAYER) return bad("unknown norm kind");
    if (p.norm_kind == B200_NORM_LAYER && p.post_norm) return bad("the layer norm is not available in the norm-after-sum form");
    if (p.streams < 0 || p.streams > ST_MAX) return bad("streams must be 0 .. " + std::to_string(ST_MAX));
    if (p.streams > 0 && (p.post_norm || looped)) return bad("the multi-stream form takes neither the norm after the sum nor a repeated range");
    if (p.parallel_ff && (p.post_norm || p.streams > 0)) return bad("parallel_ff belongs to the norm-first form with one residual stream");
    for (int i = 0; i < p.n_layers; i++) {
        const b200_layer_desc& L = layers[i];
        const std::string at = "layer " + std::to_string(i) + ": ";
        if (L.mixer == B200_MIX_WINDOW_MEMORY) {
            const b200_window_attn_desc& a = L.attn;
            const b200_matrix_memory_desc& mm = L.mem;
            if (a.heads <= 0 || a.kv_heads <= 0 || a.dim <= 0 || a.vdim <= 0 || a.kv_heads > a.heads) return bad(at + "bad attention head counts or sizes");
            if (a.window <= 0 || a.keep_first < 0) return bad(at + "window must be positive, keep_first non-negative");
            if (a.vdim > 32 * ATT_ACC) return bad(at + "attention value size above " + std::to_string(32 * ATT_ACC));
            if (mm.heads <= 0 || mm.dim <= 0 || mm.vdim <= 0 || !(mm.gate_cap > 0.0f)) return bad(at + "bad matrix-memory sizes");
            if (mm.dim > 256) return bad(at + "matrix-memory key size above 256");
        } else if (L.mixer == B200_MIX_GATED_DELTA) {
            const b200_gated_delta_desc& g = L.delta;
            if (g.heads <= 0 || g.kv_heads <= 0 || g.dim <= 0 || g.vdim <= 0 || g.kv_heads > g.heads || g.conv < 1) return bad(at + "bad delta-rule sizes");
            if (g.dim > 256) return bad(at + "delta-rule key size above 256");
        } else if (L.mixer == B200_MIX_SOFTMAX_ATTN || L.mixer == B200_MIX_ATTN_RECURRENT) {
            const b200_softmax_attn_desc& a = L.sattn;
            if (a.heads <= 0 || a.kv_heads <= 0 || a.dim <= 0 || a.vdim <= 0 || a.kv_heads > a.heads || a.heads % a.kv_heads)
                return bad(at + "bad attention head counts or sizes");
            if (a.mask != B200_MASK_WINDOW && a.mask != B200_MASK_CHUNK && a.mask != B200_MASK_CAUSAL) return bad(at + "bad attention mask");
            if (a.mask != B200_MASK_CAUSAL && a.mask_size <= 0) return bad(at + "bad attention mask");
            if (a.vdim > 32 * ATT_ACC) return bad(at + "attention value size above " + std::to_string(32 * ATT_ACC));
            if (a.rot_dims < 0 || a.rot_dims > a.dim || (a.rot_dims & 1) || (a.rot_dims > 0 && !(a.rot_base > 0.0f))) return bad(at + "bad rotary sizes");
            if (a.yarn_factor < 0.0f || (a.yarn_factor > 0.0f && !(a.yarn_original > 0.0f && a.yarn_fast > 0.0f && a.yarn_slow > 0.0f && a.rot_base > 1.0f)))
                return bad(at + "bad rotary scaling");
            if (a.v_rot_base < 0.0f || (a.v_rot_base > 0.0f && (a.vdim & 1))) return bad(at + "turned values need an even value size and a positive base");
            if (a.sink < B200_SINK_NONE || a.sink > B200_SINK_ZERO) return bad(at + "unknown sink kind");
            if (a.qk_norm < B200_QKNORM_NONE || a.qk_norm > B200_QKNORM_HEAD_UNIT) return bad(at + "unknown q/k norm");
            if (a.out_gate < B200_GATE_NONE || a.out_gate > B200_GATE_HEAD) return bad(at + "unknown output gate");
            if (a.v_mix < B200_VMIX_NONE || a.v_mix > B200_VMIX_BLEND) return bad(at + "unknown value mixing");
            if (a.conv < 0 || a.softcap < 0.0f || a.dist_bias_exp < 0.0f) return bad(at + "negative attention constant");
            if (a.v_mix == B200_VMIX_BLEND) {
                int src = -1;
                for (int j = 0; j < i; j++)
                    if (layers[j].mixer == B200_MIX_SOFTMAX_ATTN && layers[j].sattn.v_mix == B200_VMIX_SOURCE) src = j;
                if (src < 0) return bad(at + "values are blended but no earlier layer is their source");
                if (layers[src].sattn.kv_heads * layers[src].sattn.vdim != a.kv_heads * a.vdim) return bad(at + "blended values differ in size from their source");
            }
            if (looped && a.v_mix != B200_VMIX_NONE) return bad(at + "value mixing inside a program with a repeated range is not supported");
            if (L.mixer == B200_MIX_ATTN_RECURRENT) {
                if (a.v_mix != B200_VMIX_NONE) return bad(at + "the attention branch beside a recurrent unit takes no value mixing");
                if (L.rec_kind == B200_REC_GATED_LINEAR) {
                    if (L.glin.heads <= 0 || L.glin.dim <= 0 || L.glin.vdim <= 0) return bad(at + "bad gated-linear sizes");
                    if (L.glin.dim > 256) return bad(at + "gated-linear key size above 256");
                } else if (L.rec_kind == B200_REC_GATED_UNIT) {
                    if (L.gunit.width <= 0) return bad(at + "bad gated-unit width");
                } else return bad(at + "unknown recurrent unit");
                if (L.combine != B200_COMBINE_WEIGHTED && L.combine != B200_COMBINE_NORMED_MEAN) return bad(at + "unknown way to combine the branches");
                if (L.combine == B200_COMBINE_NORMED_MEAN && (p.post_norm || p.streams > 0)) return bad(at + "normed branches belong to the norm-first form with one residual stream");
            }
        } else if (L.mixer == B200_MIX_LATENT_ATTN) {
            const b200_latent_attn_desc& a = L.latent;
            if (a.heads <= 0 || a.dim <= 0 || a.rot_dim < 0 || a.vdim <= 0 || a.q_rank <= 0 || a.kv_rank <= 0) return bad(at + "bad latent-attention sizes");
            if (a.kv_rank > 32 * ATT_ACC) return bad(at + "latent size above " + std::to_string(32 * ATT_ACC));
            if (a.mask_size < 0) return bad(at + "negative window");
            if (a.rot.dims < 0 || a.rot.dims > a.rot_dim || (a.rot.dims & 1) || (a.rot.dims > 0 && !(a.rot.base > 0.0f))) return bad(at + "bad rotary sizes");
            if (a.rot.yarn_factor < 0.0f || (a.rot.yarn_factor > 0.0f && !(a.rot.yarn_original > 0.0f && a.rot.yarn_fast > 0.0f && a.rot.yarn_slow > 0.0f)))
                return bad(at + "bad rotary scaling");
            if (a.out_gate != B200_GATE_NONE && a.out_gate != B200_GATE_CHANNEL) return bad(at + "latent attention takes no gate or one per value channel");
            if (a.kv_from >= 0) {
                if (a.kv_from >= i || layers[a.kv_from].mixer != B200_MIX_LATENT_ATTN || layers[a.kv_from].latent.kv_from >= 0)
                    return bad(at + "kv_from must name an earlier latent-attention layer with cache rows of its own");
                const b200_latent_attn_desc& o = layers[a.kv_from].latent;
                if (o.kv_rank != a.kv_rank || o.rot_dim != a.rot_dim) return bad(at + "borrowed cache rows differ in size");
                if (looped) return bad(at + "borrowed cache rows inside a program with a repeated range are not supported");
            }
        } else if (L.mixer == B200_MIX_STATE_SPACE) {
            const b200_state_space_desc& g = L.ssd;
            if (g.heads <= 0 || g.vdim <= 0 || g.state <= 0 || g.groups <= 0 || g.conv < 1 || g.norm_groups <= 0) return bad(at + "bad state-space sizes");
            if (g.heads % g.groups || (g.heads * g.vdim) % g.norm_groups) return bad(at + "state-space heads / groups do not divide");
            if (g.state > 256) return bad(at + "state size above 256");
        } else return bad(at + "unknown mixer");
        if (L.ff_kind == B200_FF_MOE) {
            const b200_moe_desc& e = L.moe;
            if (e.experts <= 0 || e.top <= 0 || e.top > e.experts || e.expert_ff <= 0 || e.shared_ff < 0) return bad(at + "bad mixture-of-experts sizes");
            if (e.act < B200_ACT_RELU2 || e.act > B200_ACT_SILU_GLU || e.route < B200_ROUTE_TOP_SOFTMAX || e.route > B200_ROUTE_SIGMOID_TOP)
                return bad(at + "unknown expert activation or routing rule");
            if (e.act == B200_ACT_SILU_GLU && e.shared_ff > 0) return bad(at + "gated experts take no always-on expert");
            if (e.weight_input && p.streams > 0) return bad(at + "weights on the experts' inputs are not available in the multi-stream form");
        } else if (L.ff_kind == B200_FF_CLAMPED_GLU) {
            if (L.ff > 0 && !(L.ff_limit > 0.0f)) return bad(at + "the clamped feed-forward needs a positive limit");
        } else if (L.ff_kind != B200_FF_RELU2 && L.ff_kind != B200_FF_GATED_GELU) return bad(at + "unknown feed-forward kind");
        if (L.ff < 0) return bad(at + "negative feed-forward width");
    }
    LpModel* m = new LpModel();
    m->p = p;
    m->layers.assign(layers, layers + p.n_layers);
    m->device = device;
    m->stream = stream;
    m->f32 = p.compute == B200_COMPUTE_F32;
    m->taps_on = taps;
    // the order of layer runs: [0, start) once, [start, stop) `times` times, [stop, n) once
    auto push = [&](int li, int pass) {
        m->runs.push_back(li);
        m->run_pass.push_back(pass);
    };
    if (looped) {
        for (int i = 0; i < p.loop_start; i++) push(i, -1);
        for (int t = 0; t < p.loop_times; t++)
            for (int i = p.loop_start; i < p.loop_stop; i++) push(i, i == p.loop_start ? t : -1);
        for (int i = p.loop_stop; i < p.n_layers; i++) push(i, -1);
    } else {
        for (int i = 0; i < p.n_layers; i++) push(i, -1);
    }
    m->slot.resize(p.max_batch);
    {
        const char* e = getenv("B200_LP_TC");
        if (e && *e) m->use_tc = atoi(e) != 0;
        e = getenv("B200_LP_FUSE");
        if (e && *e) m->use_fuse = atoi(e) != 0;
        e = getenv("B200_LP_ATTN_TILE");
        if (e && *e) m->use_attn_tile = atoi(e) != 0;
        e = getenv("B200_LP_GLIN_SEG");
        if (e && *e) m->use_glin_seg = atoi(e) != 0;
        e = getenv("B200_LP_STREAM_TAIL");
        if (e && *e) m->use_stream_tail = atoi(e) != 0;
        e = getenv("B200_LP_GRAPH");
        if (e && *e) m->use_graph = atoi(e) != 0;
        e = getenv("B200_LP_TC_MIN_ROWS");
        if (e && *e) m->tc_min_rows = std::max(1, atoi(e));
    }
    *out = m;
    return B200_OK;
}

int lp_upload(LpModel* m, const char* name, uint32_t type, const uint64_t* ne, int n_dims, const void* host, size_t nbytes, std::string* err) {
    if (m->finalized) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_ctx_upload_tensor: context already finalized");
    if (n_dims < 1 || n_dims > 2) return lp_fail(err, B200_ERR_SHAPE_MISMATCH, std::string(name) + ": 1 or 2 dims expected");
    size_t es;
    if (type == B200_TYPE_BF16 || type == B200_TYPE_F16) es = 2;
    else if (type == B200_TYPE_F32) es = 4;
    else return lp_fail(err, B200_ERR_UNSUPPORTED_DTYPE, std::string(name) + ": layer-program contexts take BF16, F16 or F32 tensors");
    const uint64_t cols = ne[0], rows = n_dims == 2 ? ne[1] : 1;
    const uint64_t numel = cols * rows;
    if (numel * es != nbytes) return lp_fail(err, B200_ERR_SHAPE_MISMATCH, std::string(name) + ": byte size does not match shape");
    const std::string nm(name);
    Tensor t;
    t.matrix = is_matrix_name(nm) && n_dims == 2;
    t.rows = rows;
    t.cols = cols;
    const bool store_bf16 = t.matrix && !m->f32;
    std::vector<uint8_t> conv;
    const void* src = host;
    if (store_bf16) {
        if (type != B200_TYPE_BF16) {
            conv.resize(numel * 2);
            uint16_t* o = (uint16_t*)conv.data();
            for (uint64_t i = 0; i < numel; i++)
                o[i] = f32_to_bf16(type == B200_TYPE_F32 ? ((const float*)host)[i] : f16_to_f32(((const uint16_t*)host)[i]));
            src = conv.data();
        }
        t.bytes = numel * 2;
    } else {
        if (type != B200_TYPE_F32) {
            conv.resize(numel * 4);
            float* o = (float*)conv.data();
            for (uint64_t i = 0; i < numel; i++)
                o[i] = type == B200_TYPE_BF16 ? bf16_to_f32(((const uint16_t*)host)[i]) : f16_to_f32(((const uint16_t*)host)[i]);
            src = conv.data();
        }
        t.bytes = numel * 4;
    }
    LCU(cudaSetDevice(m->device));
    auto old = m->tensors.find(nm);
    if (old != m->tensors.end()) cudaFree(old->second.d);
    LCU_ALLOC(cudaMalloc(&t.d, up16(t.bytes)));
    LCU(cudaMemcpy(t.d, src, t.bytes, cudaMemcpyHostToDevice));
    m->tensors[nm] = t;
    return B200_OK;
}

namespace {
// Concatenate the rows of several [n_i][K] matrices into one device matrix; the pieces are freed.
int fuse_rows(LpModel* m, const std::vector<std::string>& names, const std::vector<uint64_t>& want_rows, uint64_t K, void** out, int* n_out,
              std::vector<int>* offs, std::string* err) {
    uint64_t total = 0;
    for (size_t i = 0; i < names.size(); i++) {
        const Tensor* t = find(m, names[i]);
        if (!t) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "missing tensor " + names[i]);
        if (!t->matrix || t->cols != K || t->rows != want_rows[i])
            return lp_fail(err, B200_ERR_SHAPE_MISMATCH, names[i] + ": expected [" + std::to_string(want_rows[i]) + ", " + std::to_string(K) + "], got [" +
                                                             std::to_string(t->rows) + ", " + std::to_string(t->cols) + "]");
        offs->push_back((int)total);
        total += t->rows;
    }
    void* d = nullptr;
    LCU_ALLOC(cudaMalloc(&d, up16(total * K * elt(m))));
    size_t off = 0;
    for (const std::string& n : names) {
        Tensor& t = m->tensors[n];
        LCU(cudaMemcpy((uint8_t*)d + off, t.d, t.bytes, cudaMemcpyDeviceToDevice));
        off += t.bytes;
        cudaFree(t.d);
        m->weight_bytes += t.bytes;
        m->tensors.erase(n);
    }
    *out = d;
    *n_out = (int)total;
    return B200_OK;
}
int need_vec(LpModel* m, const std::string& name, uint64_t n, const float** out, std::string* err) {
    const Tensor* t = find(m, name);
    if (!t) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "missing tensor " + name);
    if (t->matrix || t->rows * t->cols != n)
        return lp_fail(err, B200_ERR_SHAPE_MISMATCH, name + ": expected " + std::to_string(n) + " values, got " + std::to_string(t->rows * t->cols));
    *out = (const float*)t->d;
    m->weight_bytes += t->bytes;
    return B200_OK;
}
// The frequencies of the dims / 2 rotated pairs, f_i = base^(-2i / dims), stretched as b200_rotary_desc says when yarn_factor > 0;
// *gain (when asked for) receives the factor on cos and sin, 1 without stretching.
std::vector<double> rotary_frequencies(const b200_rotary_desc& ro, float* gain) {
    const int half = ro.dims / 2;
    std::vector<double> f(half);
    for (int i = 0; i < half; i++) f[i] = std::pow((double)ro.base, -2.0 * (double)i / (double)ro.dims);
    if (gain) *gain = 1.0f;
    if (ro.yarn_factor > 0.0f) {
        const double pi = 3.14159265358979323846;
        auto turn_dim = [&](double t) { return (double)ro.dims * std::log((double)ro.yarn_original / (2.0 * pi * t)) / (2.0 * std::log((double)ro.base)); };
        const double lo = std::max(std::floor(turn_dim(ro.yarn_fast)), 0.0), hi = std::min(std::ceil(turn_dim(ro.yarn_slow)), (double)ro.dims - 1.0);
        for (int i = 0; i < half; i++) {
            const double ramp = std::min(1.0, std::max(0.0, ((double)i - lo) / std::max(hi - lo, 0.001)));
            f[i] = f[i] / (double)ro.yarn_factor * ramp + f[i] * (1.0 - ramp);
        }
        if (gain) *gain = (float)(0.1 * std::log((double)ro.yarn_factor) + 1.0);
    }
    return f;
}
int need_mat(LpModel* m, const std::string& name, uint64_t rows, uint64_t cols, void** out, std::string* err) {
    const Tensor* t = find(m, name);
    if (!t) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "missing tensor " + name);
    if (!t->matrix || t->rows != rows || t->cols != cols)
        return lp_fail(err, B200_ERR_SHAPE_MISMATCH, name + ": expected [" + std::to_string(rows) + ", " + std::to_string(cols) + "], got [" +
                                                         std::to_string(t->rows) + ", " + std::to_string(t->cols) + "]");
    *out = t->d;
    m->weight_bytes += t->bytes;
    return B200_OK;
}
}  // namespace

int lp_finalize(LpModel* m, std::string* err) {
    if (m->finalized) return B200_OK;
    LCU(cudaSetDevice(m->device));
    const b200_program_desc& p = m->p;
    const uint64_t W = p.width;
    int rc;
    m->plan.resize(p.n_layers);
    void* dummy;
    if ((rc = need_mat(m, "embed", p.vocab, W, &dummy, err))) return rc;
    m->weight_bytes -= find(m, "embed")->bytes - W * elt(m);   // one row per token
    if ((rc = need_mat(m, "head", p.vocab, W, &dummy, err))) return rc;
    const float* fv;
    if ((rc = need_vec(m, "final.norm", W, &fv, err))) return rc;
    if (p.loop_stop > p.loop_start && (rc = need_vec(m, "loop.step", (uint64_t)p.loop_times * W, &fv, err))) return rc;
    for (int li = 0; li < p.n_layers; li++) {
        LayerPlan& L = m->plan[li];
        L.d = m->layers[li];
        const std::string pre = "l" + std::to_string(li) + ".";
        if ((rc = need_vec(m, pre + "norm1", W, &L.norm1, err))) return rc;
        std::vector<int> off;
        if (L.d.mixer == B200_MIX_WINDOW_MEMORY) {
            const b200_window_attn_desc& a = L.d.attn;
            const b200_matrix_memory_desc& mm = L.d.mem;
            const std::string l = pre + "mix.left.", r = pre + "mix.right.";
            std::vector<std::string> names = {l + "q", l + "k", l + "v"};
            std::vector<uint64_t> rows = {(uint64_t)a.heads * a.dim, (uint64_t)a.kv_heads * a.dim, (uint64_t)a.kv_heads * a.vdim};
            if (a.out_gate) { names.push_back(l + "g"); rows.push_back((uint64_t)a.heads * a.vdim); }
            const size_t n_left = names.size();
            for (const char* s : {"q", "k", "v", "g", "i", "f"}) names.push_back(r + s);
            for (uint64_t v : {(uint64_t)mm.heads * mm.dim, (uint64_t)mm.heads * mm.dim, (uint64_t)mm.heads * mm.vdim, (uint64_t)mm.heads * mm.vdim,
                               (uint64_t)mm.heads, (uint64_t)mm.heads})
                rows.push_back(v);
            if ((rc = fuse_rows(m, names, rows, W, &L.w_in, &L.n_in, &off, err))) return rc;
            AttnGeom& g = L.ag;
            g.H = a.heads; g.G = a.kv_heads; g.dim = a.dim; g.vdim = a.vdim; g.window = a.window; g.keep_first = a.keep_first;
            g.qk_norm = a.qk_norm; g.out_gate = a.out_gate; g.scale = a.scale; g.eps = p.norm_eps; g.cap = p.max_seq_len;
            g.q_off = off[0]; g.k_off = off[1]; g.v_off = off[2]; g.g_off = a.out_gate ? off[3] : 0;
            MemGeom& q = L.mg;
            q.H = mm.heads; q.dim = mm.dim; q.vdim = mm.vdim; q.cap = mm.gate_cap;
            q.q_off = off[n_left]; q.k_off = off[n_left + 1]; q.v_off = off[n_left + 2]; q.i_off = off[n_left + 4]; q.f_off = off[n_left + 5];
            L.dg.g_off = off[n_left + 3];   // (gate columns of the memory branch)
            if (a.qk_norm) {
                if ((rc = need_vec(m, l + "q.norm", a.dim, &L.qn, err))) return rc;
                if ((rc = need_vec(m, l + "k.norm", a.dim, &L.kn, err))) return rc;
            }
            {   // the two output projections side by side: one product [attention | memory] x [W_o attention | W_o memory]^T
                void *wa, *wm;
                const size_t Ka = (size_t)a.heads * a.vdim, Kb = (size_t)mm.heads * mm.vdim, es = elt(m);
                if ((rc = need_mat(m, l + "o", W, Ka, &wa, err))) return rc;
                if ((rc = need_mat(m, r + "o", W, Kb, &wm, err))) return rc;
                LCU_ALLOC(cudaMalloc(&L.wo_cat, up16(W * (Ka + Kb) * es)));
                LCU(cudaMemcpy2D(L.wo_cat, (Ka + Kb) * es, wa, Ka * es, Ka * es, W, cudaMemcpyDeviceToDevice));
                LCU(cudaMemcpy2D((uint8_t*)L.wo_cat + Ka * es, (Ka + Kb) * es, wm, Kb * es, Kb * es, W, cudaMemcpyDeviceToDevice));
                L.k_cat = (int)(Ka + Kb);
                for (const std::string& nm : {l + "o", r + "o"}) {
                    cudaFree(m->tensors[nm].d);
                    m->tensors.erase(nm);
                }
            }
            if ((rc = need_vec(m, r + "norm", (uint64_t)mm.heads * mm.vdim, &L.mem_norm, err))) return rc;
            if ((rc = need_vec(m, r + "i.b", mm.heads, &L.ib, err))) return rc;
            if ((rc = need_vec(m, r + "f.b", mm.heads, &L.fb, err))) return rc;
            L.kv_bytes = up16((size_t)p.max_seq_len * a.kv_heads * (a.dim + a.vdim) * 4);
            L.rec_bytes = up16(((size_t)mm.heads * mm.dim * mm.vdim + (size_t)mm.heads * mm.dim + mm.heads) * 4);
            m->max_act = std::max(m->max_act, L.k_cat);
            m->max_o = std::max(m->max_o, mm.heads * mm.vdim);
            m->max_q = std::max(m->max_q, a.heads * a.dim);
        } else if (L.d.mixer == B200_MIX_SOFTMAX_ATTN || L.d.mixer == B200_MIX_ATTN_RECURRENT) {
            // the general softmax mixer, alone ('.mix.*') or as the left branch beside a recurrent unit ('.mix.left.*', '.mix.right.*'):
            // one input projection [q | k | v | gate | the unit's projections]
            const b200_softmax_attn_desc& a = L.d.sattn;
            const bool dual = L.d.mixer == B200_MIX_ATTN_RECURRENT;
            const std::string x = pre + (dual ? "mix.left." : "mix."), rx = pre + "mix.right.";
            const uint64_t nq = (uint64_t)a.heads * a.dim, nk = (uint64_t)a.kv_heads * a.dim, nv = (uint64_t)a.kv_heads * a.vdim;
            std::vector<std::string> names = {x + "q", x + "k", x + "v"};
            std::vector<uint64_t> rows = {nq, nk, nv};
            if (a.out_gate) { names.push_back(x + "g"); rows.push_back(a.out_gate == B200_GATE_HEAD ? (uint64_t)a.heads : (uint64_t)a.heads * a.vdim); }
            const size_t n_left = names.size();
            if (dual && L.d.rec_kind == B200_REC_GATED_LINEAR) {
                const b200_gated_linear_desc& q = L.d.glin;
                for (const char* sfx : {"q", "v", "f"}) names.push_back(rx + sfx);
                for (uint64_t v : {(uint64_t)q.heads * q.dim, (uint64_t)q.heads * q.vdim, (uint64_t)q.heads * q.dim}) rows.push_back(v);
            } else if (dual) {
                for (const char* sfx : {"z", "x", "g"}) names.push_back(rx + sfx);
                for (int k = 0; k < 3; k++) rows.push_back((uint64_t)L.d.gunit.width);
            }
            if ((rc = fuse_rows(m, names, rows, W, &L.w_in, &L.n_in, &off, err))) return rc;
            AttnGeom& g = L.ag;
            g.H = a.heads; g.G = a.kv_heads; g.dim = a.dim; g.vdim = a.vdim; g.keep_first = 0;
            g.window = a.mask == B200_MASK_CAUSAL ? p.max_seq_len : a.mask_size;
            g.chunk = a.mask == B200_MASK_CHUNK ? 1 : 0; g.softcap = a.softcap; g.slope_exp = a.dist_bias_exp;
            g.qk_norm = 0; g.out_gate = a.out_gate; g.scale = a.scale; g.eps = p.norm_eps; g.cap = p.max_seq_len;
            g.q_off = off[0]; g.k_off = off[1]; g.v_off = off[2]; g.g_off = a.out_gate ? off[3] : 0;
            g.sink_mode = a.sink;
            PrepGeom& q = L.pg;
            q.C = (int)(nq + nk + nv); q.taps = a.conv; q.qk_norm = a.qk_norm; q.rot_dims = a.rot_dims; q.v_mix = a.v_mix;
            q.rot_after_norm = a.rot_after_norm; q.rot_gain = 1.0f; q.v_rot = a.v_rot_base > 0.0f ? 1 : 0;
            // concatenate per-part vectors ([q | k | v] order of the projection) into one device table; `per` values per channel
            auto cat3 = [&](const char* suffix, uint64_t per, const float** out) -> int {
                const float* part[3];
                const uint64_t n[3] = {nq * per, nk * per, nv * per};
                const char* nm[3] = {"q", "k", "v"};
                for (int i = 0; i < 3; i++)
                    if ((rc = need_vec(m, x + nm[i] + suffix, n[i], &part[i], err))) return rc;
                float* d = nullptr;
                LCU_ALLOC(cudaMalloc((void**)&d, up16((n[0] + n[1] + n[2]) * 4)));
                LCU(cudaMemcpy(d, part[0], n[0] * 4, cudaMemcpyDeviceToDevice));
                LCU(cudaMemcpy(d + n[0], part[1], n[1] * 4, cudaMemcpyDeviceToDevice));
                LCU(cudaMemcpy(d + n[0] + n[1], part[2], n[2] * 4, cudaMemcpyDeviceToDevice));
                Tensor t;
                t.d = d; t.rows = q.C; t.cols = per; t.bytes = (n[0] + n[1] + n[2]) * 4;
                m->tensors[x + "qkv" + suffix] = t;
                *out = d;
                return B200_OK;
            };
            if (a.qkv_bias && (rc = cat3(".b", 1, &L.qkv_bias))) return rc;
            if (q.taps > 0 && (rc = cat3(".conv", q.taps, &L.conv_w))) return rc;
            if (a.qk_norm == B200_QKNORM_HEAD_WEIGHT || a.qk_norm == B200_QKNORM_WHOLE_WEIGHT) {
                const bool whole = a.qk_norm == B200_QKNORM_WHOLE_WEIGHT;
                if ((rc = need_vec(m, x + "q.norm", whole ? nq : (uint64_t)a.dim, &L.qn, err))) return rc;
                if ((rc = need_vec(m, x + "k.norm", whole ? nk : (uint64_t)a.dim, &L.kn, err))) return rc;
            }
            // a table of doubles on the device, owned by the tensor map under `name`
            auto freq_table = [&](const std::vector<double>& f, const std::string& name, const double** out) -> int {
                double* d = nullptr;
                LCU_ALLOC(cudaMalloc((void**)&d, up16(f.size() * 8)));
                LCU(cudaMemcpy(d, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
                Tensor t;
                t.d = d; t.rows = 1; t.cols = f.size(); t.bytes = f.size() * 8;
                m->tensors[name] = t;
                *out = d;
                return B200_OK;
            };
            if (a.rot_dims > 0) {   // the pairs' frequencies in double, stretched when yarn_factor > 0 (b200_rotary_desc)
                const b200_rotary_desc ro{a.rot_dims, a.rot_base, a.yarn_factor, a.yarn_original, a.yarn_fast, a.yarn_slow};
                if ((rc = freq_table(rotary_frequencies(ro, &q.rot_gain), x + "rot.freq", &L.rot_freq))) return rc;
            }
            if (q.v_rot) {          // the values' own frequencies: v_rot_base^(-2m / vdim), never stretched
                const b200_rotary_desc ro{a.vdim, a.v_rot_base, 0.0f, 0.0f, 0.0f, 0.0f};
                if ((rc = freq_table(rotary_frequencies(ro, nullptr), x + "vrot.freq", &L.v_freq))) return rc;
                m->max_vrot = std::max(m->max_vrot, a.vdim);
            }
            if (a.sink == B200_SINK_LEARNED && (rc = need_vec(m, x + "sink", a.heads, &L.sink, err))) return rc;
            if (a.o_bias && (rc = need_vec(m, x + "o.b", W, &L.o_bias, err))) return rc;
            if (a.v_mix == B200_VMIX_BLEND && (rc = need_vec(m, x + "vmix", 1, &L.vmix, err))) return rc;
            L.k_left = a.heads * a.vdim;
            L.kv_bytes = up16((size_t)p.max_seq_len * (nk + nv) * 4);
            const size_t tail_bytes = q.taps > 1 ? up16((size_t)(q.taps - 1) * q.C * 4) : 0;
            L.rec_bytes = tail_bytes;
            m->max_q = std::max(m->max_q, (int)nq);
            if (a.v_mix != B200_VMIX_NONE) m->max_vsrc = std::max(m->max_vsrc, (int)nv);
            if (!dual) {
                if ((rc = need_mat(m, x + "o", W, (uint64_t)L.k_left, &L.wo, err))) return rc;
                m->max_act = std::max(m->max_act, L.k_left);
            } else {
                // the unit's state sits behind the convolution tail in the run's state block
                if (L.d.rec_kind == B200_REC_GATED_LINEAR) {
                    const b200_gated_linear_desc& u = L.d.glin;
                    GlinGeom& gg = L.gl;
                    gg.H = u.heads; gg.dim = u.dim; gg.vdim = u.vdim; gg.q_off = off[n_left]; gg.v_off = off[n_left + 1]; gg.f_off = off[n_left + 2];
                    gg.rec_off = tail_bytes;
                    if ((rc = need_vec(m, rx + "f.b", (uint64_t)u.heads * u.dim, &L.rec_b0, err))) return rc;
                    if ((rc = need_vec(m, rx + "lower", (uint64_t)u.heads * u.dim, &L.rec_lower, err))) return rc;
                    if ((rc = need_vec(m, rx + "norm", u.vdim, &L.rec_norm, err))) return rc;
                    L.k_right = u.heads * u.vdim;
                    L.rec_bytes += up16((size_t)u.heads * u.dim * u.vdim * 4);
                    m->max_o = std::max(m->max_o, L.k_right);
                } else {
                    GunitGeom& gg = L.gu;
                    gg.width = L.d.gunit.width; gg.z_off = off[n_left]; gg.x_off = off[n_left + 1]; gg.g_off = off[n_left + 2];
                    gg.rec_off = tail_bytes;
                    if ((rc = need_vec(m, rx + "z.b", gg.width, &L.rec_b0, err))) return rc;
                    if ((rc = need_vec(m, rx + "x.b", gg.width, &L.rec_b1, err))) return rc;
                    L.k_right = gg.width;
                    L.rec_bytes += up16((size_t)gg.width * 4);
                }
                L.k_cat = L.k_left + L.k_right;
                m->max_act = std::max(m->max_act, L.k_cat);
                if (L.d.combine == B200_COMBINE_WEIGHTED) {
                    // the two output projections side by side: one product [left | right] x [W_o left | W_o right]^T
                    if (a.o_bias) return lp_fail(err, B200_ERR_UNSUPPORTED, pre + "mix: an output bias with weighted branches is not supported");
                    void *wa, *wm;
                    const size_t Ka = (size_t)L.k_left, Kb = (size_t)L.k_right, es = elt(m);
                    if ((rc = need_mat(m, x + "o", W, Ka, &wa, err))) return rc;
                    if ((rc = need_mat(m, rx + "o", W, Kb, &wm, err))) return rc;
                    LCU_ALLOC(cudaMalloc(&L.wo_cat, up16(W * (Ka + Kb) * es)));
                    LCU(cudaMemcpy2D(L.wo_cat, (Ka + Kb) * es, wa, Ka * es, Ka * es, W, cudaMemcpyDeviceToDevice));
                    LCU(cudaMemcpy2D((uint8_t*)L.wo_cat + Ka * es, (Ka + Kb) * es, wm, Kb * es, Kb * es, W, cudaMemcpyDeviceToDevice));
                    for (const std::string& nm : {x + "o", rx + "o"}) {
                        cudaFree(m->tensors[nm].d);
                        m->tensors.erase(nm);
                    }
                } else {
                    if ((rc = need_mat(m, x + "o", W, (uint64_t)L.k_left, &L.wo, err))) return rc;
                    if ((rc = need_mat(m, rx + "o", W, (uint64_t)L.k_right, &L.wo_right, err))) return rc;
                    if ((rc = need_vec(m, pre + "mix.left.out", W, &L.left_out, err))) return rc;
                    if ((rc = need_vec(m, pre + "mix.right.out", W, &L.right_out, err))) return rc;
                    m->need_y2 = true;
                }
            }
        } else if (L.d.mixer == B200_MIX_LATENT_ATTN) {
            const b200_latent_attn_desc& a = L.d.latent;
            const std::string x = pre + "mix.";
            const bool own = a.kv_from < 0;
            const uint64_t H = a.heads, D = (uint64_t)a.kv_rank + a.rot_dim, per = (uint64_t)a.dim + a.rot_dim;
            std::vector<std::string> names = {x + "dq"};
            std::vector<uint64_t> rows = {(uint64_t)a.q_rank};
            if (own) { names.push_back(x + "dkv"); rows.push_back(D); }
            if (a.out_gate) { names.push_back(x + "g"); rows.push_back(H * a.vdim); }
            if ((rc = fuse_rows(m, names, rows, W, &L.w_in, &L.n_in, &off, err))) return rc;
            LatentGeom& g = L.lg;
            g.H = a.heads; g.dim = a.dim; g.rot_dim = a.rot_dim; g.vdim = a.vdim; g.q_rank = a.q_rank; g.kv_rank = a.kv_rank;
            g.rot_n = a.rot.dims; g.eps = p.norm_eps; g.cap = p.max_seq_len;
            g.q_off = off[0]; g.kv_off = own ? off[1] : -1; g.g_off = a.out_gate ? off[own ? 2 : 1] : 0;
            if ((rc = need_vec(m, x + "dq.norm", a.q_rank, &L.dq_norm, err))) return rc;
            if (own && (rc = need_vec(m, x + "dkv.norm", a.kv_rank, &L.dkv_norm, err))) return rc;
            if ((rc = need_mat(m, x + "uq", H * per, a.q_rank, &L.w_uq, err))) return rc;
            if ((rc = need_mat(m, x + "uv", H * a.vdim, a.kv_rank, &L.w_uv, err))) return rc;
            if ((rc = need_mat(m, x + "o", W, H * a.vdim, &L.wo, err))) return rc;
            {   // W_uk [H dim][kv_rank] -> per head [kv_rank][dim]: the matrix that carries a head's plain query into the latent
                void* uk;
                if ((rc = need_mat(m, x + "uk", H * a.dim, a.kv_rank, &uk, err))) return rc;
                Tensor t = *find(m, x + "uk");
                LCU_ALLOC(cudaMalloc(&t.d, up16(t.bytes)));
                const size_t n = (size_t)H * a.dim * a.kv_rank;
                if (m->f32) lp_transpose_heads_kernel<float><<<(unsigned)((n + 255) / 256), 256>>>((const float*)uk, (float*)t.d, a.heads, a.dim, a.kv_rank);
                else lp_transpose_heads_kernel<bf16><<<(unsigned)((n + 255) / 256), 256>>>((const bf16*)uk, (bf16*)t.d, a.heads, a.dim, a.kv_rank);
                LCU(cudaDeviceSynchronize());
                cudaFree(uk);
                m->tensors.erase(x + "uk");
                t.rows = H * a.kv_rank; t.cols = a.dim;
                m->tensors[x + "uk.t"] = t;
                L.w_ukT = t.d;
            }
            if (a.rot.dims > 0) {   // frequencies of the pairs, in double (see b200_rotary_desc)
                const std::vector<double> f = rotary_frequencies(a.rot, &g.rot_mult);
                double* d = nullptr;
                LCU_ALLOC(cudaMalloc((void**)&d, up16(f.size() * 8)));
                LCU(cudaMemcpy(d, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
                Tensor t;
                t.d = d; t.rows = 1; t.cols = f.size(); t.bytes = f.size() * 8;
                m->tensors[x + "rot.freq"] = t;
                L.rot_freq = d;
            }
            AttnGeom& ag = L.ag;   // the cached rows as one K/V head: keys = the whole row, values = its first kv_rank entries
            ag.H = a.heads; ag.G = 1; ag.dim = (int)D; ag.vdim = a.kv_rank; ag.window = a.mask_size > 0 ? a.mask_size : p.max_seq_len;
            ag.scale = a.scale; ag.eps = p.norm_eps; ag.cap = p.max_seq_len; ag.v_in_k = 1;
            L.kv_bytes = own ? up16((size_t)p.max_seq_len * D * 4) : 0;
            L.kv_layer = own ? li : a.kv_from;
            m->max_act = std::max(m->max_act, (int)(H * std::max(std::max(a.dim, a.kv_rank), a.vdim)));
            m->max_q = std::max(m->max_q, (int)(H * D));
            m->max_o = std::max(m->max_o, (int)(H * std::max(per, (uint64_t)a.vdim)));
            m->max_qrank = std::max(m->max_qrank, a.q_rank);
        } else if (L.d.mixer == B200_MIX_STATE_SPACE) {
            const b200_state_space_desc& g = L.d.ssd;
            const std::string x = pre + "mix.";
            const uint64_t inner = (uint64_t)g.heads * g.vdim, gn = (uint64_t)g.groups * g.state, C = inner + 2 * gn;
            L.n_in = (int)(2 * inner + 2 * gn + g.heads);
            if ((rc = need_mat(m, x + "in", L.n_in, W, &L.w_in, err))) return rc;
            m->tensors.erase(x + "in");   // (the plan owns its input projection)
            DeltaGeom& d = L.dg;          // the convolution's view: C channels from column `inner` on, the tail behind the matrix states
            d.H = g.heads; d.dim = g.state; d.vdim = g.vdim; d.taps = g.conv; d.C = (int)C; d.in_off = (int)inner;
            SsdGeom& q = L.sg;
            q.H = g.heads; q.G = g.groups; q.N = g.state; q.vdim = g.vdim; q.dt_off = (int)(inner + C);
            if ((rc = need_vec(m, x + "conv", C * g.conv, &L.conv_w, err))) return rc;
            if ((rc = need_vec(m, x + "conv.b", C, &L.conv_b, err))) return rc;
            if ((rc = need_vec(m, x + "A_log", g.heads, &L.A_log, err))) return rc;
            if ((rc = need_vec(m, x + "dt_bias", g.heads, &L.dt_bias, err))) return rc;
            if ((rc = need_vec(m, x + "D", g.heads, &L.ssd_D, err))) return rc;
            if ((rc = need_vec(m, x + "norm", inner, &L.ssd_norm, err))) return rc;
            if ((rc = need_mat(m, x + "o", W, inner, &L.wo, err))) return rc;
            L.rec_bytes = up16(((size_t)g.heads * g.state * g.vdim + (size_t)(g.conv - 1) * C) * 4);
            m->max_act = std::max(m->max_act, (int)inner);
            m->max_o = std::max(m->max_o, (int)inner);
            m->max_conv = std::max(m->max_conv, (int)C);
        } else {
            const b200_gated_delta_desc& g = L.d.delta;
            const std::string x = pre + "mix.";
            const uint64_t qk = (uint64_t)g.kv_heads * g.dim, vv = (uint64_t)g.heads * g.vdim;
            std::vector<std::string> names = {x + "q", x + "k", x + "v", x + "g", x + "b", x + "a"};
            std::vector<uint64_t> rows = {qk, qk, vv, vv, (uint64_t)g.heads, (uint64_t)g.heads};
            if ((rc = fuse_rows(m, names, rows, W, &L.w_in, &L.n_in, &off, err))) return rc;
            DeltaGeom& d = L.dg;
            d.H = g.heads; d.G = g.kv_heads; d.dim = g.dim; d.vdim = g.vdim; d.taps = g.conv; d.C = (int)(2 * qk + vv);
            d.g_off = off[3]; d.b_off = off[4]; d.a_off = off[5]; d.eps = p.norm_eps;
            // the three convolutions as one [C][taps] table in the column order of the projection
            const float *cq, *ck, *cv;
            if ((rc = need_vec(m, x + "q.conv", qk * g.conv, &cq, err))) return rc;
            if ((rc = need_vec(m, x + "k.conv", qk * g.conv, &ck, err))) return rc;
            if ((rc = need_vec(m, x + "v.conv", vv * g.conv, &cv, err))) return rc;
            float* cw = nullptr;
            LCU_ALLOC(cudaMalloc((void**)&cw, up16((size_t)d.C * g.conv * 4)));
            LCU(cudaMemcpy(cw, cq, qk * g.conv * 4, cudaMemcpyDeviceToDevice));
            LCU(cudaMemcpy(cw + qk * g.conv, ck, qk * g.conv * 4, cudaMemcpyDeviceToDevice));
            LCU(cudaMemcpy(cw + 2 * qk * g.conv, cv, vv * g.conv * 4, cudaMemcpyDeviceToDevice));
            Tensor t;
            t.d = cw; t.rows = d.C; t.cols = g.conv; t.bytes = (size_t)d.C * g.conv * 4;
            m->tensors[x + "qkv.conv"] = t;
            L.conv_w = cw;
            if ((rc = need_vec(m, x + "A_log", g.heads, &L.A_log, err))) return rc;
            if ((rc = need_vec(m, x + "dt_bias", g.heads, &L.dt_bias, err))) return rc;
            if ((rc = need_vec(m, x + "norm", g.vdim, &L.delta_norm, err))) return rc;
            if ((rc = need_mat(m, x + "o", W, vv, &L.wo_delta, err))) return rc;
            L.rec_bytes = up16(((size_t)g.heads * g.dim * g.vdim + (size_t)std::max(0, g.conv - 1) * d.C) * 4);
            m->max_act = std::max(m->max_act, (int)vv);
            m->max_o = std::max(m->max_o, (int)vv);
            m->max_conv = std::max(m->max_conv, d.C);
        }
        m->max_in = std::max(m->max_in, L.n_in);
        if (p.streams > 0) {   // the stream weights of the two sublayers; a layer without them mixes nothing
            for (int q = 0; q < 2; q++) {
                const std::string hc = pre + "hc" + std::to_string(q + 1) + ".";
                if (!find(m, hc + "in")) continue;
                if ((rc = need_vec(m, hc + "in", p.streams, &L.hc_in[q], err))) return rc;
                if ((rc = need_vec(m, hc + "out", p.streams, &L.hc_out[q], err))) return rc;
                if ((rc = need_vec(m, hc + "mix", (uint64_t)p.streams * p.streams, &L.hc_mix[q], err))) return rc;
            }
        }
        // parallel_ff: the feed-forward reads the mixer's normed input, so its first projection ([gate | up], [up] or the router) joins
        // the layer's input projection: one product per layer for everything that reads the norm; there is no second norm
        const bool par = p.parallel_ff != 0;
        auto join_input = [&](const std::vector<std::string>& names, const std::vector<uint64_t>& rows) -> int {
            void* cat = nullptr;
            int n_cat = 0;
            std::vector<int> o2;
            if ((rc = fuse_rows(m, names, rows, W, &cat, &n_cat, &o2, err))) return rc;
            void* both = nullptr;
            const size_t es = elt(m), a = (size_t)L.n_in * W * es, b = (size_t)n_cat * W * es;
            LCU_ALLOC(cudaMalloc(&both, up16(a + b)));
            LCU(cudaMemcpy(both, L.w_in, a, cudaMemcpyDeviceToDevice));
            LCU(cudaMemcpy((uint8_t*)both + a, cat, b, cudaMemcpyDeviceToDevice));
            cudaFree(L.w_in);
            cudaFree(cat);
            L.w_in = both;
            L.ff_off = L.n_in;
            L.n_in += n_cat;
            m->max_in = std::max(m->max_in, L.n_in);
            return B200_OK;
        };
        if (L.d.ff_kind == B200_FF_MOE) {
            const b200_moe_desc& e = L.d.moe;
            if (!par && (rc = need_vec(m, pre + "norm2", W, &L.norm2, err))) return rc;
            const bool glu = e.act == B200_ACT_SILU_GLU;
            const int per = glu ? 2 * e.expert_ff : e.expert_ff;   // rows of one expert's up matrix ([gate | up] when gated)
            if (par && (rc = join_input({pre + "mlp.router"}, {(uint64_t)e.experts}))) return rc;
            std::vector<std::string> names, down;
            std::vector<uint64_t> rows;
            if (!par) { names.push_back(pre + "mlp.router"); rows.push_back((uint64_t)e.experts); }
            L.up_router_rows = par ? 0 : e.experts;
            for (int i = 0; i < e.experts; i++) {
                if (glu) { names.push_back(pre + "mlp.e" + std::to_string(i) + ".gate"); rows.push_back(e.expert_ff); }
                names.push_back(pre + "mlp.e" + std::to_string(i) + ".up");
                rows.push_back(e.expert_ff);
                down.push_back(pre + "mlp.e" + std::to_string(i) + ".down");
            }
            if (e.shared_ff > 0) {
                names.push_back(pre + "mlp.shared.up");
                rows.push_back(e.shared_ff);
                down.push_back(pre + "mlp.shared.down");
            }
            std::vector<int> uoff;
            if ((rc = fuse_rows(m, names, rows, W, &L.w_up, &L.n_up, &uoff, err))) return rc;
            {
                Tensor t;
                t.d = L.w_up; t.matrix = true; t.rows = L.n_up; t.cols = W; t.bytes = (size_t)L.n_up * W * elt(m);
                m->tensors[pre + "mlp.up_cat"] = t;
            }
            // the down projections side by side: [width][e0 | e1 | ... | always-on]: one product with the weighted activations
            L.k_down = e.experts * e.expert_ff + e.shared_ff;
            const size_t es = elt(m);
            LCU_ALLOC(cudaMalloc(&L.w_down, up16(W * (size_t)L.k_down * es)));
            for (size_t i = 0; i < down.size(); i++) {
                const size_t k = i < (size_t)e.experts ? e.expert_ff : e.shared_ff;
                void* src;
                if ((rc = need_mat(m, down[i], W, k, &src, err))) return rc;
                LCU(cudaMemcpy2D((uint8_t*)L.w_down + i * e.expert_ff * es, (size_t)L.k_down * es, src, k * es, k * es, W, cudaMemcpyDeviceToDevice));
                cudaFree(m->tensors[down[i]].d);
                m->tensors.erase(down[i]);
            }
            Tensor t;
            t.d = L.w_down; t.matrix = true; t.rows = W; t.cols = L.k_down; t.bytes = W * (size_t)L.k_down * es;
            m->tensors[pre + "mlp.down_cat"] = t;
            m->max_act = std::max(m->max_act, L.k_down);
            m->max_in = std::max(m->max_in, std::max(L.n_up, e.experts * per));
            m->weight_bytes -= (size_t)(e.experts - e.top) * (per + e.expert_ff) * W * es;   // a token reads its chosen experts only
            m->max_experts = std::max(m->max_experts, e.experts);
            m->max_top = std::max(m->max_top, e.top);
        } else if (L.d.ff > 0) {
            if (!par && (rc = need_vec(m, pre + "norm2", W, &L.norm2, err))) return rc;
            const bool two = L.d.ff_kind == B200_FF_GATED_GELU || L.d.ff_kind == B200_FF_CLAMPED_GLU;
            if (par) {
                if (two) rc = join_input({pre + "mlp.gate", pre + "mlp.up"}, {(uint64_t)L.d.ff, (uint64_t)L.d.ff});
                else rc = join_input({pre + "mlp.up"}, {(uint64_t)L.d.ff});
                if (rc) return rc;
                L.n_up = two ? 2 * L.d.ff : L.d.ff;
            } else if (two) {
                std::vector<int> uoff;
                if ((rc = fuse_rows(m, {pre + "mlp.gate", pre + "mlp.up"}, {(uint64_t)L.d.ff, (uint64_t)L.d.ff}, W, &L.w_up, &L.n_up, &uoff, err))) return rc;
                Tensor t;
                t.d = L.w_up; t.matrix = true; t.rows = L.n_up; t.cols = W; t.bytes = (size_t)L.n_up * W * elt(m);
                m->tensors[pre + "mlp.gate_up"] = t;
                m->max_in = std::max(m->max_in, L.n_up);
            } else {
                if ((rc = need_mat(m, pre + "mlp.up", L.d.ff, W, &L.w_up, err))) return rc;
                L.n_up = L.d.ff;
            }
            if ((rc = need_mat(m, pre + "mlp.down", W, L.d.ff, &L.w_down, err))) return rc;
            L.k_down = L.d.ff;
            m->max_act = std::max(m->max_act, L.d.ff);
        } else if (p.post_norm && find(m, pre + "norm2")) {   // a layer without feed-forward whose file still holds the second norm
            if ((rc = need_vec(m, pre + "norm2", W, &L.norm2, err))) return rc;
        }
    }
    {   // the preparation kernel of the softmax mixer keeps a row's q, k, v in shared memory
        size_t need = 0;
        for (const LayerPlan& L : m->plan)
            if (L.d.mixer == B200_MIX_SOFTMAX_ATTN || L.d.mixer == B200_MIX_ATTN_RECURRENT)
                need = std::max(need, (size_t)(((L.pg.C + 3) & ~3) + L.pg.rot_dims + (L.pg.v_rot ? L.ag.vdim : 0)) * 4);
        if (need > 200 * 1024) return lp_fail(err, B200_ERR_UNSUPPORTED, "softmax mixer: q, k and v of one token exceed 200 KB of shared memory");
        if (need > 32 * 1024) LCU(cudaFuncSetAttribute(lp_attn_prep2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need));
    }
    if (p.norm_weight_offset != 0.0f) {   // norm weights stored around zero: (offset + w) once, in f32
        std::vector<std::string> nm = {"final.norm"};
        for (int li = 0; li < p.n_layers; li++)
            for (const char* s2 : {".norm1", ".norm2"}) nm.push_back("l" + std::to_string(li) + s2);
        for (const std::string& n : nm) {
            const Tensor* t = find(m, n);
            if (t) lp_add_scalar_kernel<<<(unsigned)((t->rows * t->cols + 255) / 256), 256>>>((float*)t->d, (int)(t->rows * t->cols), p.norm_weight_offset);
        }
        LCU(cudaDeviceSynchronize());
    }
    // layout of a slot: cache block (all runs with attention) and state block (all runs)
    size_t kv = 0, rec = 0;
    for (size_t r = 0; r < m->runs.size(); r++) {
        const LayerPlan& L = m->plan[m->runs[r]];
        m->run_kv_off.push_back(kv);
        m->run_rec_off.push_back(rec);
        kv += L.kv_bytes;
        rec += L.rec_bytes;
        m->weight_bytes += 0;
        if (L.d.mixer == B200_MIX_WINDOW_MEMORY) m->kv_bytes_per_pos += (size_t)L.d.attn.kv_heads * (L.d.attn.dim + L.d.attn.vdim) * 4;
        if (L.d.mixer == B200_MIX_SOFTMAX_ATTN || L.d.mixer == B200_MIX_ATTN_RECURRENT)
            m->kv_bytes_per_pos += (size_t)L.d.sattn.kv_heads * (L.d.sattn.dim + L.d.sattn.vdim) * 4;
        if (L.d.mixer == B200_MIX_LATENT_ATTN && L.d.latent.kv_from < 0) m->kv_bytes_per_pos += (size_t)(L.d.latent.kv_rank + L.d.latent.rot_dim) * 4;
    }
    m->slot_kv_bytes = std::max<size_t>(kv, 256);
    m->slot_rec_bytes = std::max<size_t>(rec, 256);
    // frequencies of the sinusoidal position vector, in double
    {
        const int nf = (p.width + 1) / 2;
        std::vector<double> f(nf);
        for (int i = 0; i < nf; i++) f[i] = std::pow(10000.0, -2.0 * (double)i / (double)p.width);
        LCU_ALLOC(cudaMalloc((void**)&m->inv_freq, up16(nf * sizeof(double))));
        LCU(cudaMemcpy(m->inv_freq, f.data(), nf * sizeof(double), cudaMemcpyHostToDevice));
    }
    if (p.streams > 0) {   // the stream kernel keeps a row of the width in shared memory
        if ((size_t)p.width * 4 > 200 * 1024) return lp_fail(err, B200_ERR_UNSUPPORTED, "multi-stream form: a row exceeds 200 KB of shared memory");
        if ((size_t)p.width * 4 > 32 * 1024) {
            const int sb = p.width * 4;
            LCU(cudaFuncSetAttribute(lp_streams_kernel<float, 1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<float, 4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<bf16, 1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<bf16, 4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<float, 1, ST_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<float, 4, ST_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<bf16, 1, ST_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
            LCU(cudaFuncSetAttribute(lp_streams_kernel<bf16, 4, ST_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb));
        }
    }
    LCU_ALLOC(cudaMalloc((void**)&m->tc_err, 256));
    LCU(cudaMemset(m->tc_err, 0, 256));
    m->tail_counter = (unsigned*)(m->tc_err + 16);
    LCU_ALLOC(cudaHostAlloc((void**)&m->h_tc_err, 64, cudaHostAllocDefault));
    *m->h_tc_err = 0;
    m->finalized = true;
    return B200_OK;
}

void lp_destroy(LpModel* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    cudaStreamSynchronize(m->stream);
    for (auto& kv : m->tensors) cudaFree(kv.second.d);
    for (auto& g : m->graphs)
        if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    for (LayerPlan& L : m->plan) {
        cudaFree(L.w_in);
        cudaFree(L.wo_cat);
    }
    for (SlotMem& s : m->slot) { cudaFree(s.kv); cudaFree(s.rec); }
    for (SlotMem& s : m->pool) { cudaFree(s.kv); cudaFree(s.rec); }
    for (void* ptr : {(void*)m->inv_freq, (void*)m->d_meta, (void*)m->x, (void*)m->P, (void*)m->qbuf, (void*)m->O, (void*)m->conv, (void*)m->logits,
                      m->hn, m->act_a, m->hw, (void*)m->pick, (void*)m->taps, (void*)m->glin_carry, (void*)m->y, (void*)m->vsrc, (void*)m->moe_w, (void*)m->moe_selw,
                      (void*)m->moe_sel, (void*)m->moe_pos, (void*)m->moe_seg, m->moe_xp, (void*)m->moe_yp, (void*)m->xs, m->cq, (void*)m->vrot})
        cudaFree(ptr);
    if (m->h_meta) cudaFreeHost(m->h_meta);
    if (m->h_logits) cudaFreeHost(m->h_logits);
    if (m->h_tc_err) cudaFreeHost(m->h_tc_err);
    cudaFree(m->tc_err);
    delete m;
}

int lp_layer_runs(const LpModel* m) { return (int)m->runs.size(); }

void lp_stats(const LpModel* m, uint64_t* launches, uint64_t* weight_bytes, uint64_t* kv_bytes_per_pos) {
    if (launches) *launches = m->launches;
    if (weight_bytes) *weight_bytes = m->weight_bytes;
    if (kv_bytes_per_pos) *kv_bytes_per_pos = m->kv_bytes_per_pos;
}

void lp_pool_counts(const LpModel* m, int* live, int* pooled) {
    int n = 0;
    for (const SlotMem& s : m->slot) n += s.rec != nullptr;
    if (live) *live = n;
    if (pooled) *pooled = (int)m->pool.size();
}

int lp_release(LpModel* m, int seq, std::string* err) {
    if (seq < 0 || seq >= (int)m->slot.size()) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "bad sequence slot");
    if (m->slot[seq].rec) {
        m->pool.push_back(m->slot[seq]);
        m->slot[seq] = SlotMem();
    }
    return B200_OK;
}

int lp_get_taps(LpModel* m, float* out, size_t cap_floats, std::string* err) {
    if (!m->taps_on) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_get_taps: taps are off (B200_TAPS=1 before the context is created)");
    const size_t n = (size_t)m->runs.size() * m->taps_len * m->p.width;
    if (!out || cap_floats < n) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_get_taps: buffer too small");
    LCU(cudaSetDevice(m->device));
    LCU(cudaMemcpy(out, m->taps, n * 4, cudaMemcpyDeviceToHost));
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ the step
namespace {
template <typename P>
int grow(P** ptr, size_t bytes, std::string* err) {
    cudaFree(*ptr);
    *ptr = nullptr;
    LCU_ALLOC(cudaMalloc((void**)ptr, up16(bytes)));
    return B200_OK;
}

int ensure_scratch(LpModel* m, int R, int n_runs, int n_want, std::string* err) {
    int rc;
    if (R > m->cap_rows || n_want > m->cap_want || n_runs > m->cap_runs) m->scratch_epoch++;   // buffers or table offsets move: graphs are void
    const size_t es = elt(m);
    const int W = m->p.width;
    if (R > m->cap_rows) {
        const int cap = std::max(R, std::min(2 * m->cap_rows, 1 << 20));
        if ((rc = grow(&m->x, (size_t)cap * W * 4, err))) return rc;
        if ((rc = grow(&m->P, (size_t)cap * m->max_in * 4, err))) return rc;
        if ((rc = grow(&m->qbuf, (size_t)cap * std::max(m->max_q, 1) * 4, err))) return rc;
        if ((rc = grow(&m->O, (size_t)cap * std::max(m->max_o, 1) * 4, err))) return rc;
        if ((rc = grow(&m->conv, (size_t)cap * std::max(m->max_conv, 1) * 4, err))) return rc;
        if ((rc = grow(&m->hn, (size_t)cap * W * es, err))) return rc;
        if ((rc = grow(&m->act_a, (size_t)cap * m->max_act * es, err))) return rc;
        if ((m->p.post_norm || m->max_experts > 0 || m->p.streams > 0 || m->need_y2) && (rc = grow(&m->y, (size_t)cap * W * (m->need_y2 ? 8 : 4), err))) return rc;
        if (m->max_vrot > 0 && (rc = grow(&m->vrot, (size_t)cap * m->max_vrot * 4, err))) return rc;
        if (m->p.streams > 0 && (rc = grow(&m->xs, (size_t)cap * m->p.streams * W * 4, err))) return rc;
        if (m->max_qrank > 0 && (rc = grow(&m->cq, (size_t)cap * m->max_qrank * es, err))) return rc;
        if (m->max_vsrc > 0 && (rc = grow(&m->vsrc, (size_t)cap * m->max_vsrc * 4, err))) return rc;
        if (m->max_experts > 0) {
            if ((rc = grow(&m->moe_w, (size_t)cap * m->max_experts * 4, err))) return rc;
            if ((rc = grow(&m->moe_selw, (size_t)cap * m->max_top * 4, err))) return rc;
            if ((rc = grow(&m->moe_sel, (size_t)cap * m->max_top * 4, err))) return rc;
            if ((rc = grow(&m->moe_pos, (size_t)cap * m->max_top * 4, err))) return rc;
            if ((rc = grow(&m->moe_seg, (size_t)(2 * m->max_experts + 2) * 4, err))) return rc;
            if ((rc = grow(&m->moe_xp, (size_t)cap * m->max_top * W * es, err))) return rc;
            if ((rc = grow(&m->moe_yp, (size_t)cap * m->max_top * W * 4, err))) return rc;
        }
        m->cap_rows = cap;
    }
    if (n_want > m->cap_want) {
        const int cap = std::max(n_want, 2 * m->cap_want);
        if ((rc = grow(&m->logits, (size_t)cap * m->p.vocab * 4, err))) return rc;
        if ((rc = grow(&m->hw, (size_t)cap * W * es, err))) return rc;
        if ((rc = grow(&m->pick, (size_t)cap * 4, err))) return rc;
        m->cap_want = cap;
    }
    m->cap_runs = std::max(m->cap_runs, n_runs);
    const size_t meta = up16((size_t)(3 * m->cap_rows + 2 * m->cap_runs + 2 + m->cap_want) * 4) + (size_t)2 * m->cap_runs * 8 + 64;
    if (meta > m->meta_bytes) {
        if (m->h_meta) cudaFreeHost(m->h_meta);
        m->h_meta = nullptr;
        LCU_ALLOC(cudaHostAlloc((void**)&m->h_meta, meta, cudaHostAllocDefault));
        if ((rc = grow(&m->d_meta, meta, err))) return rc;
        m->meta_bytes = meta;
    }
    return B200_OK;
}

// Tensor-pipe attention for prompt rows: bf16 mode, runs of at least 16 rows, key size a multiple of 16 up to 128, value size a
// multiple of 8 up to 256 (with 16-byte aligned cache rows); everything else takes the warp kernel.
template <int DK, int DV>
bool attn_tile_launch(LpModel* m, const StepMeta& sm, const AttnGeom& ag, int ldp, int n_runs, int max_len) {
    const size_t smem = (size_t)(AT_K * (DK + 8) + DV * (AT_K + 8)) * 2;
    static bool once[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !once[dev]) {
        if (cudaFuncSetAttribute(lp_window_attn_tile_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (dev >= 0 && dev < 64) once[dev] = true;
    }
    launch(m, lp_window_attn_tile_kernel<DK, DV>, dim3((max_len + AT_Q - 1) / AT_Q, ag.H, n_runs), dim3(128), smem, sm, ag, (const float*)m->qbuf,
           (const float*)m->P, ldp, (bf16*)m->act_a);
    return true;
}
bool attn_tile(LpModel* m, const StepMeta& sm, const AttnGeom& ag, int ldp, int n_runs, int max_len) {
    if (m->f32 || !m->use_attn_tile || max_len < 16) return false;
    if (ag.dim % 16 || ag.vdim % 8 || ag.dim > 128 || ag.vdim > 256 || ag.out_ld % 2) return false;
    if (ag.dim <= 64 && ag.vdim <= 64) return attn_tile_launch<64, 64>(m, sm, ag, ldp, n_runs, max_len);
    if (ag.vdim <= 128) return attn_tile_launch<128, 128>(m, sm, ag, ldp, n_runs, max_len);
    return attn_tile_launch<128, 256>(m, sm, ag, ldp, n_runs, max_len);
}

// Into how many segments the gated linear memory cuts the runs of a step (1 = whole runs): only long runs, and only while whole runs
// would leave SMs idle (a block per 16 to 64 columns of a head's state and run); segments of at least 64 tokens.
int glin_segments(const LpModel* m, int H, int dim, int vdim, int n_runs, int max_len) {
    if (!m->use_glin_seg || max_len < 256) return 1;
    const int cols = SCAN_BD / (pick_dmax(dim) / SCAN_DREG);
    const long blocks = (long)((vdim + cols - 1) / cols) * H * n_runs;
    if (blocks > 148) return 1;   // (measured: from one block per SM on, the segments' second pass costs what their overlap wins)
    const long want = (6 * 148 + blocks - 1) / blocks;
    return (int)std::max<long>(1, std::min<long>(std::min<long>(want, GC_SEG_MAX), max_len / 64));
}

// The warp kernel: any row count, both compute modes.
void attn_rows(LpModel* m, const StepMeta& sm, const AttnGeom& ag, const LayerPlan& L, int R) {
    dim3 agrid(R, ag.H);
    const size_t asmem = (size_t)(((ag.dim + 3) & ~3) + ATT_WARPS * ag.vdim + 2 * ATT_WARPS + (ag.vrot ? ag.vdim : 0)) * 4;
    const int vch = ag.vdim <= 128 ? 4 : ag.vdim <= 256 ? 8 : 16;
#define LP_ATTN(T, V) launch(m, lp_window_attn_kernel<T, V>, agrid, dim3(32 * ATT_WARPS), asmem, sm, ag, (const float*)m->qbuf, (const float*)m->P, L.n_in, L.qn, L.kn, (T*)m->act_a)
    if (m->f32) {
        if (vch == 4) LP_ATTN(float, 4); else if (vch == 8) LP_ATTN(float, 8); else LP_ATTN(float, 16);
    } else {
        if (vch == 4) LP_ATTN(bf16, 4); else if (vch == 8) LP_ATTN(bf16, 8); else LP_ATTN(bf16, 16);
    }
#undef LP_ATTN
}

// Every kernel of one step, in order, on the model's stream: eagerly, or while the stream is being captured into a CUDA graph (a
// decode step: one row per run, nothing allocated).  head: 0 = no logits, 1 = logits of the wanted rows, 2 = their greedy picks.
void enqueue_step(LpModel* m, const StepMeta& sm, int R, int n_runs, int n_want, int head, int taps_len, int max_len) {
    const b200_program_desc& p = m->p;
    const int W = p.width;
    const float* loop_step = p.loop_stop > p.loop_start ? (const float*)find(m, "loop.step")->d : nullptr;
    // embedding
    if (m->f32) launch(m, lp_embed_kernel<float>, dim3(R), dim3(128), 0, sm, (const float*)find(m, "embed")->d, m->inv_freq, m->x, W, p.embed_scale, p.pos_sinusoid);
    else launch(m, lp_embed_kernel<bf16>, dim3(R), dim3(128), 0, sm, (const bf16*)find(m, "embed")->d, m->inv_freq, m->x, W, p.embed_scale, p.pos_sinusoid);
    // The two layer forms.  Norm first: a sublayer reads norm(x) and its output projection adds into x.  Norm after the sum
    // (post_norm): a sublayer reads x itself -- m->hn holds x in the compute type -- its output projection goes to m->y, and
    // lp_postnorm_kernel makes x <- norm(alpha x + y) and the next copy.
    // Multi-stream form (p.streams >= 1): the copies live in m->xs; a sublayer's output goes to m->y and waits in `pend` until the
    // next sublayer (or the head) asks for its input: lp_streams_kernel then updates the copies and norms their weighted sum into m->hn.
    const bool post = p.post_norm != 0, streams = p.streams > 0;
    struct {
        const float *y, *mix, *out;
        bool src;
    } pend = {nullptr, nullptr, nullptr, true};
    // Few rows (decoding): the kernel that writes m->y also does what follows it -- its last block updates the copies and norms the
    // next input, and when a mixture comes next it routes (rows_tail); the next call of `boundary` then finds its work done.
    // (one block works through the rows one after the other: measured level with the separate launch for one row, 20 % behind it for
    // eight, so only the smallest steps take it)
    const bool sfew = streams && m->use_fuse && m->use_stream_tail && R <= 2 && taps_len == 0;
    bool pre_done = false;
    auto boundary = [&](const float* in, const float* w, float* sum) {
        if (pre_done) {
            pre_done = false;
            pend = {nullptr, nullptr, nullptr, false};
            return;
        }
        StreamStep st{};
        st.S = p.streams; st.width = W; st.src = pend.src ? m->x : nullptr; st.y = pend.y; st.mix = pend.mix; st.out = pend.out;
        st.mult = p.residual_mult; st.in = in; st.w = w; st.center = norm_center(m); st.eps = p.norm_eps; st.sum = sum;
        const bool v4 = W % 4 == 0 && (!sum || ((uintptr_t)sum & 15) == 0), few_s = p.streams <= 4;
#define LP_ST(T, V, SM) launch(m, lp_streams_kernel<T, V, SM>, dim3(R), dim3(256), (size_t)W * 4, m->xs, st, (T*)m->hn)
        if (m->f32) {
            if (v4 && few_s) LP_ST(float, 4, 4); else if (v4) LP_ST(float, 4, ST_MAX); else if (few_s) LP_ST(float, 1, 4); else LP_ST(float, 1, ST_MAX);
        } else {
            if (v4 && few_s) LP_ST(bf16, 4, 4); else if (v4) LP_ST(bf16, 4, ST_MAX); else if (few_s) LP_ST(bf16, 1, 4); else LP_ST(bf16, 1, ST_MAX);
        }
#undef LP_ST
        pend = {nullptr, nullptr, nullptr, false};
    };
    const LayerPlan* cur = nullptr;   // the layer and the sublayer (0 mixer, 1 feed-forward) that project_in / project_out serve
    int sub = 0;
    size_t cur_run = 0;
    bool cur_moe_sel = false;
    // the tail of the kernel that ends sublayer `sub` of the current layer: what the sublayer after it reads
    auto stream_tail = [&]() {
        RowsTail t{};
        t.on = 1; t.streams = 1; t.xs = m->xs; t.xc = m->hn; t.width = W; t.R = R; t.counter = m->tail_counter;
        StreamStep& st = t.st;
        st.S = p.streams; st.width = W; st.y = m->y; st.mix = cur->hc_mix[sub]; st.out = cur->hc_out[sub]; st.mult = p.residual_mult;
        st.center = norm_center(m); st.eps = p.norm_eps;
        const bool has_ff = cur->d.ff_kind == B200_FF_MOE || cur->d.ff > 0;
        if (sub == 0 && has_ff) {
            st.in = cur->hc_in[1]; st.w = cur->norm2;
            if (cur->d.ff_kind == B200_FF_MOE && cur_moe_sel) {
                const b200_moe_desc& e = cur->d.moe;
                t.router = cur->w_up; t.E = e.experts; t.top = e.top; t.route = e.route; t.route_scale = e.route_scale;
                t.logits = m->P; t.wts = m->moe_w; t.sel = m->moe_sel; t.selw = m->moe_selw;
            }
        } else if (cur_run + 1 < m->runs.size()) {
            const LayerPlan& nx = m->plan[m->runs[cur_run + 1]];
            st.in = nx.hc_in[0]; st.w = nx.norm1;
        } else st.sum = m->x;   // the head reads the sum of the copies
        return t;
    };
    auto cast_x = [&](const float* y, const float* w) {
        if (m->f32) launch(m, lp_postnorm_kernel<float>, dim3(R), dim3(256), 0, m->x, y, w, (float*)m->hn, W, p.residual_alpha, p.norm_eps);
        else launch(m, lp_postnorm_kernel<bf16>, dim3(R), dim3(256), 0, m->x, y, w, (bf16*)m->hn, W, p.residual_alpha, p.norm_eps);
    };
    auto project_in = [&](const float* add, const float* nw, const void* Wm, int N, void* Y, int ldy, int epi) {
        if (streams) {
            boundary(cur->hc_in[sub], nw, nullptr);
            gemm(m, m->hn, W, Wm, N, W, Y, ldy, R, 1.0f, epi);
        } else if (post) gemm(m, m->hn, W, Wm, N, W, Y, ldy, R, 1.0f, epi);
        else norm_gemm(m, m->x, add, nullptr, nw, m->hn, Wm, N, Y, ldy, R, 1.0f, epi, p.parallel_ff != 0);   // (parallel_ff: the experts read m->hn later)
    };
    // Few rows (decoding) in the norm-after-sum form: the kernel that writes m->y also does what follows it -- its last block norms the
    // rows and, when `moe` follows, computes the router's logits and choices (rows_tail) -- instead of two or three more launches.
    const bool few = post && m->use_fuse && R <= 2 * GV_ROWS;
    auto make_tail = [&](const float* nw, const LayerPlan* moe) {
        RowsTail t{};
        t.on = 1; t.x = m->x; t.y = m->y; t.w = nw; t.xc = m->hn; t.width = W; t.R = R; t.alpha = p.residual_alpha; t.eps = p.norm_eps;
        t.counter = m->tail_counter;
        if (moe) {
            t.router = moe->w_up; t.E = moe->d.moe.experts; t.top = moe->d.moe.top; t.route = moe->d.moe.route; t.route_scale = moe->d.moe.route_scale;
            t.logits = m->P; t.wts = m->moe_w; t.sel = m->moe_sel; t.selw = m->moe_selw;
        }
        return t;
    };
    auto project_out = [&](const void* X, int K, const void* Wm, const float* nw, const LayerPlan* moe, const float* bias = nullptr) {
        if (sfew) {
            const RowsTail t = stream_tail();
            gemm(m, X, K, Wm, W, K, m->y, W, R, 1.0f, EPI_STORE, &t, bias);
            pre_done = true;
        } else if (streams) {
            gemm(m, X, K, Wm, W, K, m->y, W, R, 1.0f, EPI_STORE, nullptr, bias);
            pend.y = m->y; pend.mix = cur->hc_mix[sub]; pend.out = cur->hc_out[sub];
        } else if (few) {
            const RowsTail t = make_tail(nw, moe);
            gemm(m, X, K, Wm, W, K, m->y, W, R, 1.0f, EPI_STORE, &t, bias);
        } else if (post) {
            gemm(m, X, K, Wm, W, K, m->y, W, R, 1.0f, EPI_STORE, nullptr, bias);
            cast_x(m->y, nw);
        } else gemm(m, X, K, Wm, W, K, m->x, W, R, 1.0f, EPI_ADD, nullptr, bias);
    };
    if (post) cast_x(nullptr, nullptr);
    for (size_t run = 0; run < m->runs.size(); run++) {
        LayerPlan& L = m->plan[m->runs[run]];
        const float* add = m->run_pass[run] >= 0 ? loop_step + (size_t)m->run_pass[run] * W : nullptr;
        // the few-row expert kernels (16-byte loads: sizes multiples of 8 / 4, the rows in shared memory)
        const bool moe_sel_ok = L.d.ff_kind == B200_FF_MOE && m->use_fuse && R <= 2 * GV_ROWS && W % (m->f32 ? 4 : 8) == 0 &&
                                L.d.moe.expert_ff % (m->f32 ? 4 : 8) == 0 && L.d.moe.shared_ff % (m->f32 ? 4 : 8) == 0 && (size_t)R * W * elt(m) <= 40 * 1024;
        const LayerPlan* moe_next = ((few || sfew) && moe_sel_ok) ? &L : nullptr;      // the mixer's output kernel also routes
        cur = &L;
        sub = 0;
        cur_run = run;
        cur_moe_sel = moe_sel_ok;
        project_in(add, L.norm1, L.w_in, L.n_in, m->P, L.n_in, EPI_STORE);
        if (L.d.mixer == B200_MIX_SOFTMAX_ATTN || L.d.mixer == B200_MIX_ATTN_RECURRENT) {
            const bool dual = L.d.mixer == B200_MIX_ATTN_RECURRENT, weighted = dual && L.d.combine == B200_COMBINE_WEIGHTED;
            AttnGeom ag = L.ag;
            ag.kv_off = m->run_kv_off[run];
            ag.out_ld = dual ? L.k_cat : L.k_left;          // the two branches' operands side by side: [left | right]
            ag.out_scale = weighted ? L.d.attn_scale : 1.0f;
            ag.fused_prep = 0;
            ag.sink = L.sink;
            ag.vrot = L.pg.v_rot ? m->vrot : nullptr;
            PrepGeom pg = L.pg;
            pg.rec_off = m->run_rec_off[run];
            const size_t psmem = (size_t)(((pg.C + 3) & ~3) + pg.rot_dims + (pg.v_rot ? ag.vdim : 0)) * 4;
            const int shift = (m->use_fuse && max_len == 1) ? 1 : 0;   // one row per run: the row's block moves the run's tail on itself
            launch(m, lp_attn_prep2_kernel, dim3(R), dim3(256), psmem, sm, ag, pg, (const float*)m->P, L.n_in, L.qkv_bias, L.conv_w, L.qn, L.kn, L.rot_freq,
                   L.vmix, m->vsrc, m->qbuf, shift, L.v_freq, m->vrot);
            if (pg.taps > 1 && !shift) launch(m, lp_attn_conv_tail_kernel, dim3(n_runs), dim3(256), 0, sm, pg, (const float*)m->P, L.n_in, L.qkv_bias);
            if (!attn_tile(m, sm, ag, L.n_in, n_runs, max_len)) attn_rows(m, sm, ag, L, R);
            if (!dual) {
                project_out(m->act_a, ag.out_ld, L.wo, L.norm1, moe_next, L.o_bias);
            } else {
                const size_t es = elt(m);
                void* right = (uint8_t*)m->act_a + (size_t)L.k_left * es;      // the unit's output, column k_left on
                const float rscale = weighted ? L.d.mem_scale : 1.0f;
                if (L.d.rec_kind == B200_REC_GATED_LINEAR) {
                    GlinGeom gg = L.gl;
                    gg.rec_off += m->run_rec_off[run];
                    const int ldo = gg.H * gg.vdim;
                    const int cols = SCAN_BD / (pick_dmax(gg.dim) / SCAN_DREG);
                    dim3 sgrid((gg.vdim + cols - 1) / cols, gg.H, n_runs);
                    const int vec4 = (gg.dim % 4 == 0 && gg.q_off % 4 == 0 && gg.f_off % 4 == 0 && L.n_in % 4 == 0) ? 1 : 0;
                    launch(m, lp_glin_gates_kernel, dim3((unsigned)(((size_t)R * gg.H * gg.dim + 255) / 256)), dim3(256), 0, m->P, L.n_in, gg, L.rec_b0, L.rec_lower, R);
                    int nseg = glin_segments(m, gg.H, gg.dim, gg.vdim, n_runs, max_len);
                    if ((size_t)n_runs * nseg * gg.H * gg.dim * gg.vdim * 4 > m->glin_carry_bytes) nseg = 1;
#define LP_GLIN(DM, MODE, Z) launch(m, lp_gated_linear_kernel<DM, MODE>, dim3(sgrid.x, sgrid.y, (unsigned)(Z)), dim3(SCAN_BD), 0, sm, gg, (const float*)m->P, L.n_in, vec4, m->O, ldo, nseg, m->glin_carry)
#define LP_GLIN_ALL(MODE, Z)                                                                                           \
                    switch (pick_dmax(gg.dim)) {                                                                       \
                        case 32: LP_GLIN(32, MODE, Z); break;                                                          \
                        case 64: LP_GLIN(64, MODE, Z); break;                                                          \
                        case 128: LP_GLIN(128, MODE, Z); break;                                                        \
                        default: LP_GLIN(256, MODE, Z); break;                                                         \
                    }
                    if (nseg <= 1) {
                        LP_GLIN_ALL(0, n_runs)
                    } else {   // segments fold side by side, their carries are chained, every segment runs from its true start
                        LP_GLIN_ALL(1, n_runs * (nseg - 1))
                        launch(m, lp_glin_carry_kernel, dim3(((gg.dim + GC_CH - 1) / GC_CH) * ((gg.vdim + GC_CH - 1) / GC_CH), gg.H, n_runs), dim3(GC_CH * GC_TL), 0, sm, gg, (const float*)m->P, L.n_in, nseg, m->glin_carry);
                        LP_GLIN_ALL(2, n_runs * nseg)
                    }
#undef LP_GLIN_ALL
#undef LP_GLIN
                    dim3 hgrid(R, (gg.H + 3) / 4);   // per-head unit RMS times the shared weight, no gate
                    if (m->f32) launch(m, lp_headnorm_gate_kernel<float>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, 0, L.rec_norm, 1, gg.H, gg.vdim, p.norm_eps, 2, (float*)right, L.k_cat, rscale, R);
                    else launch(m, lp_headnorm_gate_kernel<bf16>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, 0, L.rec_norm, 1, gg.H, gg.vdim, p.norm_eps, 2, (bf16*)right, L.k_cat, rscale, R);
                } else {
                    GunitGeom gg = L.gu;
                    gg.rec_off += m->run_rec_off[run];
                    dim3 ugrid((gg.width + GU_CH - 1) / GU_CH, n_runs), ublock(GU_CH, GU_SEG);
                    if (m->f32) launch(m, lp_gated_unit_kernel<float>, ugrid, ublock, 0, sm, gg, (const float*)m->P, L.n_in, L.rec_b0, L.rec_b1, (float*)right, L.k_cat, rscale);
                    else launch(m, lp_gated_unit_kernel<bf16>, ugrid, ublock, 0, sm, gg, (const float*)m->P, L.n_in, L.rec_b0, L.rec_b1, (bf16*)right, L.k_cat, rscale);
                }
                if (weighted) {
                    project_out(m->act_a, L.k_cat, L.wo_cat, L.norm1, moe_next);
                } else {
                    // each branch through its own output projection, rms norm with its plain weight, half the sum: the sublayer's output
                    float* ya = m->y;
                    float* yb = m->y + (size_t)R * W;
                    // (norm-first form only: the sum goes straight into the residual stream)
                    gemm_ld(m, m->act_a, L.k_cat, L.wo, L.k_left, W, L.k_left, ya, W, R, EPI_STORE, L.o_bias);
                    gemm_ld(m, right, L.k_cat, L.wo_right, L.k_right, W, L.k_right, yb, W, R, EPI_STORE);
                    launch(m, lp_dual_norm_add_kernel, dim3(R), dim3(256), 0, m->x, (const float*)ya, (const float*)yb, W, L.left_out, L.right_out, W, p.norm_eps, 0.5f);
                }
            }
        } else if (L.d.mixer == B200_MIX_WINDOW_MEMORY) {
            AttnGeom ag = L.ag;
            ag.kv_off = m->run_kv_off[run];
            ag.out_ld = L.k_cat;
            ag.out_scale = L.d.attn_scale;
            ag.fused_prep = (m->use_fuse && max_len == 1) ? 1 : 0;
            if (!ag.fused_prep) launch(m, lp_attn_prep_kernel, dim3(R), dim3(128), 0, sm, ag, (const float*)m->P, L.n_in, L.qn, L.kn, m->qbuf);
            if (!attn_tile(m, sm, ag, L.n_in, n_runs, max_len)) attn_rows(m, sm, ag, L, R);
            MemGeom mg = L.mg;
            mg.rec_off = m->run_rec_off[run];
            const int ldo = mg.H * mg.vdim;
            const int mcols = SCAN_BD / (pick_dmax(mg.dim) / SCAN_DREG);
            dim3 sgrid((mg.vdim + mcols - 1) / mcols, mg.H, n_runs);
            switch (pick_dmax(mg.dim)) {
                case 32: launch(m, lp_matrix_memory_kernel<32>, sgrid, dim3(SCAN_BD), 0, sm, mg, (const float*)m->P, L.n_in, L.ib, L.fb, m->O, ldo); break;
                case 64: launch(m, lp_matrix_memory_kernel<64>, sgrid, dim3(SCAN_BD), 0, sm, mg, (const float*)m->P, L.n_in, L.ib, L.fb, m->O, ldo); break;
                case 128: launch(m, lp_matrix_memory_kernel<128>, sgrid, dim3(SCAN_BD), 0, sm, mg, (const float*)m->P, L.n_in, L.ib, L.fb, m->O, ldo); break;
                default: launch(m, lp_matrix_memory_kernel<256>, sgrid, dim3(SCAN_BD), 0, sm, mg, (const float*)m->P, L.n_in, L.ib, L.fb, m->O, ldo); break;
            }
            dim3 hgrid(R, (mg.H + 3) / 4);
            if (m->f32) launch(m, lp_headnorm_gate_kernel<float>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, L.dg.g_off, L.mem_norm, 0, mg.H, mg.vdim, p.norm_eps, 0, (float*)m->act_a + ag.H * ag.vdim, L.k_cat, L.d.mem_scale, R);
            else launch(m, lp_headnorm_gate_kernel<bf16>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, L.dg.g_off, L.mem_norm, 0, mg.H, mg.vdim, p.norm_eps, 0, (bf16*)m->act_a + ag.H * ag.vdim, L.k_cat, L.d.mem_scale, R);
            project_out(m->act_a, L.k_cat, L.wo_cat, L.norm1, moe_next);
        } else if (L.d.mixer == B200_MIX_LATENT_ATTN) {
            // P = [W_dq h | W_dkv h | W_g h] -> norms, the cache row -> q = W_uq c_q -> rotated part and W_uk^T q_plain into qbuf ->
            // attention over the cached rows (one shared K/V head, values inside the keys) -> W_uv per head -> gate -> W_o
            const b200_latent_attn_desc& a = L.d.latent;
            LatentGeom lg = L.lg;
            lg.cache_off = m->run_kv_off[L.kv_layer == m->runs[run] ? run : (size_t)L.kv_layer];
            const size_t csm = (size_t)lg.rot_n * 4;
            const int per = a.dim + a.rot_dim, D = a.kv_rank + a.rot_dim, nv = a.heads * a.vdim;
            if (m->f32) launch(m, lp_latent_prep_kernel<float>, dim3(R), dim3(256), csm, sm, lg, (const float*)m->P, L.n_in, L.dq_norm, L.dkv_norm, L.rot_freq, (float*)m->cq);
            else launch(m, lp_latent_prep_kernel<bf16>, dim3(R), dim3(256), csm, sm, lg, (const float*)m->P, L.n_in, L.dq_norm, L.dkv_norm, L.rot_freq, (bf16*)m->cq);
            gemm(m, m->cq, a.q_rank, L.w_uq, a.heads * per, a.q_rank, m->O, a.heads * per, R, 1.0f, EPI_STORE);
            if (m->f32) launch(m, lp_latent_qprep_kernel<float>, dim3(R), dim3(256), csm, sm, lg, (const float*)m->O, L.rot_freq, (float*)m->act_a, m->qbuf);
            else launch(m, lp_latent_qprep_kernel<bf16>, dim3(R), dim3(256), csm, sm, lg, (const float*)m->O, L.rot_freq, (bf16*)m->act_a, m->qbuf);
            gemm_heads(m, m->act_a, a.heads * a.dim, a.dim, L.w_ukT, a.heads, a.kv_rank, a.dim, m->qbuf, a.heads * D, D, R);
            AttnGeom ag = L.ag;
            ag.kv_off = lg.cache_off;
            ag.out_ld = a.heads * a.kv_rank;
            ag.out_scale = 1.0f;
            ag.fused_prep = 0;
            if (!attn_tile(m, sm, ag, L.n_in, n_runs, max_len)) attn_rows(m, sm, ag, L, R);
            gemm_heads(m, m->act_a, a.heads * a.kv_rank, a.kv_rank, L.w_uv, a.heads, a.vdim, a.kv_rank, m->O, nv, a.vdim, R);
            const unsigned nb = (unsigned)(((size_t)R * nv + 255) / 256);
            if (m->f32) launch(m, lp_latent_gate_kernel<float>, dim3(nb), dim3(256), 0, (const float*)m->O, (const float*)m->P, L.n_in, lg.g_off, a.out_gate, nv, R, (float*)m->act_a);
            else launch(m, lp_latent_gate_kernel<bf16>, dim3(nb), dim3(256), 0, (const float*)m->O, (const float*)m->P, L.n_in, lg.g_off, a.out_gate, nv, R, (bf16*)m->act_a);
            project_out(m->act_a, nv, L.wo, L.norm1, moe_next);
        } else if (L.d.mixer == B200_MIX_STATE_SPACE) {
            const b200_state_space_desc& g = L.d.ssd;
            DeltaGeom dg = L.dg;
            dg.rec_off = m->run_rec_off[run];
            const int shift = (m->use_fuse && max_len == 1) ? 1 : 0;
            launch(m, lp_conv_silu_kernel, dim3(R, (dg.C + 255) / 256), dim3(256), 0, sm, dg, (const float*)m->P, L.n_in, L.conv_w, L.conv_b, m->conv, shift);
            if (dg.taps > 1 && !shift) launch(m, lp_conv_tail_kernel, dim3(n_runs, (dg.C + 255) / 256), dim3(256), 0, sm, dg, (const float*)m->P, L.n_in);
            SsdGeom sg = L.sg;
            sg.rec_off = dg.rec_off;
            const int inner = g.heads * g.vdim;
            const int dcols = SCAN_BD / (pick_dmax(g.state) / SCAN_DREG);
            dim3 sgrid((g.vdim + dcols - 1) / dcols, g.heads, n_runs);
#define LP_SSD(DM) launch(m, lp_ssd_scan_kernel<DM>, sgrid, dim3(SCAN_BD), 0, sm, sg, (const float*)m->conv, dg.C, (const float*)m->P, L.n_in, L.A_log, L.dt_bias, L.ssd_D, m->O, inner)
            switch (pick_dmax(g.state)) {
                case 32: LP_SSD(32); break;
                case 64: LP_SSD(64); break;
                case 128: LP_SSD(128); break;
                default: LP_SSD(256); break;
            }
#undef LP_SSD
            if (m->f32) launch(m, lp_gate_groupnorm_kernel<float>, dim3(R, g.norm_groups), dim3(256), 0, (const float*)m->O, inner, (const float*)m->P, L.n_in, 0, L.ssd_norm, inner, g.norm_groups, p.norm_eps, (float*)m->act_a);
            else launch(m, lp_gate_groupnorm_kernel<bf16>, dim3(R, g.norm_groups), dim3(256), 0, (const float*)m->O, inner, (const float*)m->P, L.n_in, 0, L.ssd_norm, inner, g.norm_groups, p.norm_eps, (bf16*)m->act_a);
            project_out(m->act_a, inner, L.wo, L.norm1, moe_next);
        } else {
            DeltaGeom dg = L.dg;
            dg.rec_off = m->run_rec_off[run];
            const int shift = (m->use_fuse && max_len == 1) ? 1 : 0;
            launch(m, lp_conv_silu_kernel, dim3(R, (dg.C + 255) / 256), dim3(256), 0, sm, dg, (const float*)m->P, L.n_in, L.conv_w, (const float*)nullptr, m->conv, shift);
            if (dg.taps > 1 && !shift) launch(m, lp_conv_tail_kernel, dim3(n_runs, (dg.C + 255) / 256), dim3(256), 0, sm, dg, (const float*)m->P, L.n_in);
            const int ldo = dg.H * dg.vdim;
            const int dcols = SCAN_BD / (pick_dmax(dg.dim) / SCAN_DREG);
            dim3 sgrid((dg.vdim + dcols - 1) / dcols, dg.H, n_runs);
            switch (pick_dmax(dg.dim)) {
                case 32: launch(m, lp_gated_delta_kernel<32>, sgrid, dim3(SCAN_BD), 0, sm, dg, (const float*)m->conv, (const float*)m->P, L.n_in, L.A_log, L.dt_bias, m->O, ldo); break;
                case 64: launch(m, lp_gated_delta_kernel<64>, sgrid, dim3(SCAN_BD), 0, sm, dg, (const float*)m->conv, (const float*)m->P, L.n_in, L.A_log, L.dt_bias, m->O, ldo); break;
                case 128: launch(m, lp_gated_delta_kernel<128>, sgrid, dim3(SCAN_BD), 0, sm, dg, (const float*)m->conv, (const float*)m->P, L.n_in, L.A_log, L.dt_bias, m->O, ldo); break;
                default: launch(m, lp_gated_delta_kernel<256>, sgrid, dim3(SCAN_BD), 0, sm, dg, (const float*)m->conv, (const float*)m->P, L.n_in, L.A_log, L.dt_bias, m->O, ldo); break;
            }
            dim3 hgrid(R, (dg.H + 3) / 4);
            if (m->f32) launch(m, lp_headnorm_gate_kernel<float>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, dg.g_off, L.delta_norm, 1, dg.H, dg.vdim, p.norm_eps, 1, (float*)m->act_a, ldo, 1.0f, R);
            else launch(m, lp_headnorm_gate_kernel<bf16>, hgrid, dim3(128), 0, (const float*)m->O, ldo, (const float*)m->P, L.n_in, dg.g_off, L.delta_norm, 1, dg.H, dg.vdim, p.norm_eps, 1, (bf16*)m->act_a, ldo, 1.0f, R);
            project_out(m->act_a, ldo, L.wo_delta, L.norm1, moe_next);
        }
        const bool par = p.parallel_ff != 0;
        if (L.d.ff_kind == B200_FF_MOE) {
            // The operand is m->hn in every layer form; the router's rows come first in w_up ([router | e0 up | ... | always-on up]) or,
            // with parallel_ff, sit in the layer's input projection (their logits are columns ff_off .. of m->P already).
            // Router logits (f32) -> the choice per row -> the experts -> m->y -> the residual.
            const b200_moe_desc& e = L.d.moe;
            const size_t es = elt(m);
            const int act_epi = e.act == B200_ACT_GELU ? EPI_GELU : EPI_RELU2;
            const int per = e.act == B200_ACT_SILU_GLU ? 2 * e.expert_ff : e.expert_ff;      // rows of one expert's up matrix
            const bool own_act = e.act == B200_ACT_SILU_GLU || e.weight_input != 0;            // the hidden units need a kernel of their own
            sub = 1;
            if (streams) boundary(L.hc_in[1], L.norm2, nullptr);
            else if (!post && !par) rmsnorm(m, m->x, nullptr, L.norm2, m->hn, nullptr, R);
            if (par) {
                launch(m, lp_moe_route_kernel, dim3((R + 3) / 4), dim3(128), 0, (const float*)m->P + L.ff_off, L.n_in, e.experts, e.top, m->moe_w, m->moe_sel, m->moe_selw, R, e.route, e.route_scale);
            } else if (!moe_next) {
                gemm(m, m->hn, W, L.w_up, e.experts, W, m->P, e.experts, R, 1.0f, EPI_STORE);
                launch(m, lp_moe_route_kernel, dim3((R + 3) / 4), dim3(128), 0, (const float*)m->P, e.experts, e.experts, e.top, m->moe_w, m->moe_sel, m->moe_selw, R, e.route, e.route_scale);
            }
            const size_t hbytes = (size_t)R * W * es;
            const uint8_t* up_experts = (const uint8_t*)L.w_up + (size_t)L.up_router_rows * W * es;
            float* ydst = par ? m->x : m->y;          // parallel_ff: the experts' sum goes straight into the residual stream
            bool normed = false;
            if (moe_sel_ok) {
                // few rows (decoding): kernels that walk each row's choices and read those experts' weights only
                const int per_row = e.top * e.expert_ff + e.shared_ff;
                dim3 ugrid(std::min((R * per_row + 7) / 8, 8 * 148)), dgrid(std::min((R * W + 1) / 2, 8 * 148));
                const RowsTail t = sfew ? stream_tail() : few ? make_tail(L.norm2, nullptr) : RowsTail{};
                normed = few || sfew;
                if (sfew) pre_done = true;
                if (m->f32) {
                    launch(m, lp_moe_up_sel_kernel<float>, ugrid, dim3(256), hbytes, (const float*)m->hn, (const float*)up_experts, (const int*)m->moe_sel, (const float*)m->moe_selw, e.experts, e.top, e.expert_ff, e.shared_ff, W, R, (float*)m->act_a, e.act, e.weight_input);
                    launch(m, lp_moe_down_sel_kernel<float>, dgrid, dim3(256), 0, (const float*)m->act_a, (const float*)L.w_down, (const int*)m->moe_sel, e.experts, e.top, e.expert_ff, e.shared_ff, W, R, ydst, t, par ? 1 : 0);
                } else {
                    launch(m, lp_moe_up_sel_kernel<bf16>, ugrid, dim3(256), hbytes, (const bf16*)m->hn, (const bf16*)up_experts, (const int*)m->moe_sel, (const float*)m->moe_selw, e.experts, e.top, e.expert_ff, e.shared_ff, W, R, (bf16*)m->act_a, e.act, e.weight_input);
                    launch(m, lp_moe_down_sel_kernel<bf16>, dgrid, dim3(256), 0, (const bf16*)m->act_a, (const bf16*)L.w_down, (const int*)m->moe_sel, e.experts, e.top, e.expert_ff, e.shared_ff, W, R, ydst, t, par ? 1 : 0);
                }
            } else if (m->use_fuse && R > 2 * GV_ROWS) {
                // many rows: the (token, choice) pairs in expert order, one product pair per expert over its block of rows (the row
                // counts stay on the device), the always-on expert over all rows, then the weighted sum per token
                const int pairs = R * e.top;
                launch(m, lp_moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * e.experts * 4, (const int*)m->moe_sel, pairs, e.experts, m->moe_seg, m->moe_pos);
                if (m->f32) launch(m, lp_moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, (const float*)m->hn, (const int*)m->moe_pos, e.top, W, (float*)m->moe_xp);
                else launch(m, lp_moe_gather_kernel<bf16>, dim3(pairs), dim3(128), 0, (const bf16*)m->hn, (const int*)m->moe_pos, e.top, W, (bf16*)m->moe_xp);
                const uint8_t* down = (const uint8_t*)L.w_down;
                uint8_t* act_sh = (uint8_t*)m->act_a + (size_t)pairs * e.expert_ff * es;     // the always-on expert's activations behind the others
                if (own_act) {
                    // pre-activations in f32 (m->P: its router columns have been read), then the units with the pair's weight
                    gemm_grouped(m, m->moe_xp, W, up_experts, W, (size_t)per * W, e.experts, per, W, m->P, per, R, EPI_STORE, m->moe_seg);
                    const unsigned nb = (unsigned)(((size_t)pairs * e.expert_ff + 255) / 256);
                    if (m->f32) launch(m, lp_moe_pair_act_kernel<float>, dim3(nb), dim3(256), 0, (const float*)m->P, per, (const int*)m->moe_pos, (const float*)m->moe_selw, e.expert_ff, (float*)m->act_a, pairs, e.act, e.weight_input);
                    else launch(m, lp_moe_pair_act_kernel<bf16>, dim3(nb), dim3(256), 0, (const float*)m->P, per, (const int*)m->moe_pos, (const float*)m->moe_selw, e.expert_ff, (bf16*)m->act_a, pairs, e.act, e.weight_input);
                } else {
                    gemm_grouped(m, m->moe_xp, W, up_experts, W, (size_t)e.expert_ff * W, e.experts, e.expert_ff, W, m->act_a, e.expert_ff, R, act_epi, m->moe_seg);
                }
                gemm_grouped(m, m->act_a, e.expert_ff, down, L.k_down, (size_t)e.expert_ff, e.experts, W, e.expert_ff, m->moe_yp, W, R, EPI_STORE, m->moe_seg);
                if (e.shared_ff > 0) {
                    gemm(m, m->hn, W, up_experts + (size_t)e.experts * per * W * es, e.shared_ff, W, act_sh, e.shared_ff, R, 1.0f, act_epi);
                    gemm_ld(m, act_sh, e.shared_ff, down + (size_t)e.experts * e.expert_ff * es, L.k_down, W, e.shared_ff, ydst, W, R, par ? EPI_ADD : EPI_STORE);
                }
                launch(m, lp_moe_combine_kernel, dim3(R), dim3(256), 0, (const float*)m->moe_yp, (const int*)m->moe_pos, own_act ? (const float*)nullptr : (const float*)m->moe_selw, e.top, W,
                       (par || e.shared_ff > 0) ? 1 : 0, ydst);
            } else {
                // the plain form: every expert's up projection for every row, activations times their expert's weight (0 for experts
                // that were not chosen), one product with the down matrices side by side
                const int n_exp = L.n_up - L.up_router_rows;
                gemm(m, m->hn, W, up_experts, n_exp, W, m->P, n_exp, R, 1.0f, EPI_STORE);
                const unsigned nb = (unsigned)(((size_t)R * L.k_down + 255) / 256);
                if (m->f32) launch(m, lp_moe_act_kernel<float>, dim3(nb), dim3(256), 0, (const float*)m->P, n_exp, 0, (const float*)m->moe_w, e.experts, e.expert_ff, L.k_down, (float*)m->act_a, R, e.act, e.weight_input);
                else launch(m, lp_moe_act_kernel<bf16>, dim3(nb), dim3(256), 0, (const float*)m->P, n_exp, 0, (const float*)m->moe_w, e.experts, e.expert_ff, L.k_down, (bf16*)m->act_a, R, e.act, e.weight_input);
                gemm(m, m->act_a, L.k_down, L.w_down, W, L.k_down, ydst, W, R, 1.0f, par ? EPI_ADD : EPI_STORE);
            }
            if (normed || par) {
            } else if (streams) {
                pend.y = m->y; pend.mix = L.hc_mix[1]; pend.out = L.hc_out[1];
            } else if (post) cast_x(m->y, L.norm2);
            else launch(m, lp_add_rows_kernel, dim3((unsigned)(((size_t)R * W + 255) / 256)), dim3(256), 0, m->x, (const float*)m->y, (size_t)R * W);
        } else if (L.d.ff > 0 && (L.d.ff_kind == B200_FF_GATED_GELU || L.d.ff_kind == B200_FF_CLAMPED_GLU)) {
            // [gate | up] in one product (with parallel_ff: columns ff_off .. of the layer's input projection), the gated units, W_down
            sub = 1;
            const float* ffP = m->P;
            int ff_ld = L.n_up;
            if (par) { ffP = m->P + L.ff_off; ff_ld = L.n_in; }
            else project_in(nullptr, L.norm2, L.w_up, L.n_up, m->P, L.n_up, EPI_STORE);
            const unsigned nb = (unsigned)(((size_t)R * L.d.ff + 255) / 256);
            if (L.d.ff_kind == B200_FF_CLAMPED_GLU) {
                const bool v4 = L.d.ff % 4 == 0 && ff_ld % 4 == 0 && ((uintptr_t)ffP & 15) == 0;
                const unsigned nb4 = (unsigned)(((size_t)R * (L.d.ff / 4) + 255) / 256);
                if (m->f32) {
                    if (v4) launch(m, lp_clamped_glu_kernel<float, 4>, dim3(nb4), dim3(256), 0, ffP, ff_ld, (float*)m->act_a, L.d.ff, R, L.d.ff_limit, L.d.ff_slope);
                    else launch(m, lp_clamped_glu_kernel<float, 1>, dim3(nb), dim3(256), 0, ffP, ff_ld, (float*)m->act_a, L.d.ff, R, L.d.ff_limit, L.d.ff_slope);
                } else {
                    if (v4) launch(m, lp_clamped_glu_kernel<bf16, 4>, dim3(nb4), dim3(256), 0, ffP, ff_ld, (bf16*)m->act_a, L.d.ff, R, L.d.ff_limit, L.d.ff_slope);
                    else launch(m, lp_clamped_glu_kernel<bf16, 1>, dim3(nb), dim3(256), 0, ffP, ff_ld, (bf16*)m->act_a, L.d.ff, R, L.d.ff_limit, L.d.ff_slope);
                }
            } else {
                if (m->f32) launch(m, lp_gated_gelu_kernel<float>, dim3(nb), dim3(256), 0, ffP, ff_ld, (float*)m->act_a, L.d.ff, R);
                else launch(m, lp_gated_gelu_kernel<bf16>, dim3(nb), dim3(256), 0, ffP, ff_ld, (bf16*)m->act_a, L.d.ff, R);
            }
            project_out(m->act_a, L.d.ff, L.w_down, L.norm2, nullptr);
        } else if (L.d.ff > 0 && par) {
            // relu^2 of the feed-forward's columns of the layer's input projection
            sub = 1;
            const unsigned nb = (unsigned)(((size_t)R * L.d.ff + 255) / 256);
            if (m->f32) launch(m, lp_relu2_kernel<float>, dim3(nb), dim3(256), 0, (const float*)m->P + L.ff_off, L.n_in, (float*)m->act_a, L.d.ff, R);
            else launch(m, lp_relu2_kernel<bf16>, dim3(nb), dim3(256), 0, (const float*)m->P + L.ff_off, L.n_in, (bf16*)m->act_a, L.d.ff, R);
            project_out(m->act_a, L.d.ff, L.w_down, L.norm2, nullptr);
        } else if (L.d.ff > 0) {
            sub = 1;
            project_in(nullptr, L.norm2, L.w_up, L.d.ff, m->act_a, L.d.ff, EPI_RELU2);
            project_out(m->act_a, L.d.ff, L.w_down, L.norm2, nullptr);
        } else if (post && L.norm2) {
            cast_x(nullptr, L.norm2);
        }
        if (streams && taps_len > 0) boundary(nullptr, nullptr, m->x);   // the taps are the sum of the copies
        if (taps_len > 0) cudaMemcpyAsync(m->taps + run * (size_t)taps_len * W, m->x, (size_t)taps_len * W * 4, cudaMemcpyDeviceToDevice, m->stream);
    }
    if (streams) boundary(nullptr, nullptr, m->x);   // the head reads the sum of the copies
    if (head) {
        norm_gemm(m, m->x, nullptr, sm.want, (const float*)find(m, "final.norm")->d, m->hw, find(m, "head")->d, p.vocab, m->logits, p.vocab, n_want,
                  p.logit_scale, EPI_STORE);
        if (head == 2) launch(m, lp_argmax_kernel, dim3(n_want), dim3(1024), 0, (const float*)m->logits, p.vocab, m->pick);
    }
}
}  // namespace

int lp_step(LpModel* m, int n_runs, const int* seqs, const int* pos0, const int* lens, const uint32_t* tokens, const int* want_rows, int n_want,
            float* logits_out, uint32_t* pick_out, std::string* err) {
    if (!m->finalized) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: context not finalized");
    if (n_runs <= 0 || !seqs || !lens || !tokens || !pos0) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: bad argument");
    if (n_want < 0 || (n_want > 0 && !want_rows)) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: bad want_rows");
    const b200_program_desc& p = m->p;
    int R = 0;
    for (int i = 0; i < n_runs; i++) {
        if (seqs[i] < 0 || seqs[i] >= (int)m->slot.size()) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: bad sequence slot");
        for (int j = 0; j < i; j++)
            if (seqs[i] == seqs[j]) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: duplicate sequence slot");
        if (lens[i] <= 0) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: empty token run");
        if ((int64_t)pos0[i] + lens[i] > p.max_seq_len) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: context length exceeded");
        R += lens[i];
    }
    for (int r = 0; r < R; r++)
        if (tokens[r] >= (uint32_t)p.vocab) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: token id " + std::to_string(tokens[r]) + " exceeds vocab size");
    for (int i = 0; i < n_want; i++)
        if (want_rows[i] < 0 || want_rows[i] >= R) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: want_rows out of range");
    LCU(cudaSetDevice(m->device));
    int rc;
    if ((rc = ensure_scratch(m, R, n_runs, n_want, err))) return rc;
    // slot memory: a slot at position 0 starts from a zeroed state block (out of the pool when one is waiting there)
    for (int i = 0; i < n_runs; i++) {
        SlotMem& s = m->slot[seqs[i]];
        if (pos0[i] == 0 && s.rec) {   // (a slot that was rewound without a release)
            m->pool.push_back(s);
            s = SlotMem();
        }
        if (!s.rec) {
            if (pos0[i] != 0) return lp_fail(err, B200_ERR_INVALID_ARGUMENT, "b200_step: the slot holds no state for its position");
            if (!m->pool.empty()) {
                s = m->pool.back();
                m->pool.pop_back();
            } else {
                LCU_ALLOC(cudaMalloc((void**)&s.kv, m->slot_kv_bytes));
                cudaError_t e = cudaMalloc((void**)&s.rec, m->slot_rec_bytes);
                if (e != cudaSuccess) {
                    cudaFree(s.kv);
                    s = SlotMem();
                    return lp_fail(err, B200_ERR_ALLOCATION_FAILED, std::string("slot state: ") + cudaGetErrorString(e));
                }
            }
            LCU(cudaMemsetAsync(s.rec, 0, m->slot_rec_bytes, m->stream));
        }
    }
    // tables of the step
    StepMeta sm{};
    {
        int* hi = (int*)m->h_meta;
        int* tok = hi;
        int* row_run = tok + m->cap_rows;
        int* row_pos = row_run + m->cap_rows;
        int* run_start = row_pos + m->cap_rows;
        int* run_p0 = run_start + m->cap_runs + 1;
        int* want = run_p0 + m->cap_runs + 1;
        const size_t ints = up16((size_t)(3 * m->cap_rows + 2 * m->cap_runs + 2 + m->cap_want) * 4);
        uint8_t** kvp = (uint8_t**)(m->h_meta + ints);
        uint8_t** recp = kvp + m->cap_runs;
        int r = 0;
        for (int i = 0; i < n_runs; i++) {
            run_start[i] = r;
            run_p0[i] = pos0[i];
            kvp[i] = m->slot[seqs[i]].kv;
            recp[i] = m->slot[seqs[i]].rec;
            for (int t = 0; t < lens[i]; t++, r++) {
                tok[r] = (int)tokens[r];
                row_run[r] = i;
                row_pos[r] = pos0[i] + t;
            }
        }
        run_start[n_runs] = r;
        for (int i = 0; i < n_want; i++) want[i] = want_rows[i];
        LCU(cudaMemcpyAsync(m->d_meta, m->h_meta, m->meta_bytes, cudaMemcpyHostToDevice, m->stream));
        const uint8_t* d = m->d_meta;
        sm.tok = (const int*)d;
        sm.row_run = sm.tok + m->cap_rows;
        sm.row_pos = sm.row_run + m->cap_rows;
        sm.run_start = sm.row_pos + m->cap_rows;
        sm.run_pos0 = sm.run_start + m->cap_runs + 1;
        sm.want = sm.run_pos0 + m->cap_runs + 1;
        sm.run_kv = (uint8_t* const*)(d + ints);
        sm.run_rec = sm.run_kv + m->cap_runs;
    }
    const int W = p.width;
    if (m->taps_on) {
        const size_t need = (size_t)m->runs.size() * lens[0] * W;
        if (need > m->taps_floats) {
            if ((rc = grow(&m->taps, need * 4, err))) return rc;
            m->taps_floats = need;
        }
        m->taps_len = lens[0];
    }
    int max_len = 1;
    for (int i = 0; i < n_runs; i++) max_len = std::max(max_len, lens[i]);
    {   // segment carries of the gated linear memories, when this step's runs are cut
        size_t need = 0;
        for (const LayerPlan& L : m->plan)
            if (L.d.mixer == B200_MIX_ATTN_RECURRENT && L.d.rec_kind == B200_REC_GATED_LINEAR) {
                const int nseg = glin_segments(m, L.gl.H, L.gl.dim, L.gl.vdim, n_runs, max_len);
                if (nseg > 1) need = std::max(need, (size_t)n_runs * nseg * L.gl.H * L.gl.dim * L.gl.vdim * 4);
            }
        if (need > m->glin_carry_bytes) {
            m->glin_carry_bytes = 0;
            if ((rc = grow(&m->glin_carry, need, err))) return rc;
            m->glin_carry_bytes = need;
        }
    }
    const int head = (n_want > 0 && pick_out) ? 2 : (n_want > 0 && logits_out) ? 1 : 0;
    const int taps_len = m->taps_on ? lens[0] : 0;
    // A decode step (one row per run, every slot already holds state) always launches the same kernels with the same arguments: the
    // tables of the step live at fixed device addresses.  It is captured once per (rows, wanted rows, head) into a CUDA graph and
    // replayed; the first step of a shape runs eagerly (it also warms the kernels up), the second is the capture.
    bool decode = m->use_graph && !m->taps_on && R == n_runs;
    for (int i = 0; i < n_runs && decode; i++) decode = pos0[i] > 0;
    if (decode) {
        const uint64_t key = ((uint64_t)R << 34) | ((uint64_t)n_want << 4) | (uint64_t)head;
        LpModel::Graph& g = m->graphs[key];
        if (g.exec && g.epoch != m->scratch_epoch) {
            cudaGraphExecDestroy(g.exec);
            g = LpModel::Graph();
        }
        if (g.exec) {
            LCU(cudaGraphLaunch(g.exec, m->stream));
            m->launches += g.launches;
        } else if (!g.warm) {
            g.warm = true;
            enqueue_step(m, sm, R, n_runs, n_want, head, 0, 1);
        } else {
            const uint64_t before = m->launches;
            cudaGraph_t graph = nullptr;
            LCU(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
            enqueue_step(m, sm, R, n_runs, n_want, head, 0, 1);
            cudaError_t e = cudaStreamEndCapture(m->stream, &graph);
            if (e == cudaSuccess) e = cudaGraphInstantiate(&g.exec, graph, 0);
            if (graph) cudaGraphDestroy(graph);
            if (e != cudaSuccess) {
                cudaGetLastError();
                m->launch_fail.clear();
                g = LpModel::Graph();
                m->use_graph = false;          // fall back to eager launches for good
                m->launches = before;
                enqueue_step(m, sm, R, n_runs, n_want, head, 0, 1);
            } else {
                g.launches = m->launches - before;
                g.epoch = m->scratch_epoch;
                LCU(cudaGraphLaunch(g.exec, m->stream));
            }
        }
    } else {
        enqueue_step(m, sm, R, n_runs, n_want, head, taps_len, max_len);
    }
    if (head == 2) {
        LCU(cudaMemcpyAsync(pick_out, m->pick, (size_t)n_want * 4, cudaMemcpyDeviceToHost, m->stream));
    } else if (head == 1) {
        const size_t bytes = (size_t)n_want * p.vocab * 4;
        if (bytes > m->h_logits_bytes) {
            if (m->h_logits) cudaFreeHost(m->h_logits);
            m->h_logits = nullptr;
            m->h_logits_bytes = 0;
            LCU_ALLOC(cudaHostAlloc((void**)&m->h_logits, bytes, cudaHostAllocDefault));
            m->h_logits_bytes = bytes;
        }
        LCU(cudaMemcpyAsync(m->h_logits, m->logits, bytes, cudaMemcpyDeviceToHost, m->stream));
    }
    LCU(cudaMemcpyAsync(m->h_tc_err, m->tc_err, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    LCU(cudaStreamSynchronize(m->stream));
    {
        const cudaError_t e_ = cudaGetLastError();
        if (e_ != cudaSuccess || !m->launch_fail.empty()) {
            const std::string what = m->launch_fail.empty() ? std::string(cudaGetErrorString(e_)) : m->launch_fail;
            m->launch_fail.clear();
            return lp_fail(err, B200_ERR_OPERATION_FAILED, "b200_step: " + what);
        }
    }
    if (*m->h_tc_err) {   // a bounded wait of the tensor-core GEMM gave up: the step's results are void
        const int code = *m->h_tc_err;
        *m->h_tc_err = 0;
        cudaMemset(m->tc_err, 0, sizeof(int));
        return lp_fail(err, B200_ERR_OPERATION_FAILED, "b200_step: tensor-core GEMM wait gave up (code " + std::to_string(code) + "): results discarded");
    }
    if (n_want > 0 && logits_out) memcpy(logits_out, m->h_logits, (size_t)n_want * p.vocab * 4);
    return B200_OK;
}
