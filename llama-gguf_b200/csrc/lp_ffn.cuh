// lp_ffn.cuh — the norm-after-sum layer form and the feed-forward kinds beside relu^2: the gated tanh-GELU layer and the mixture of
// experts (router, top-k weights, expert activations).  Included by layerprog.cu inside its anonymous namespace.
#pragma once

// x <- (alpha x + y) / sqrt(mean((alpha x + y)^2) + eps) * w, kept in f32; xc receives the same row in the compute type (the
// sublayers of such a layer read x itself, so this copy is the next GEMM's operand).  w = null: x is only copied (the embedding);
// y = null: nothing is added.
template <typename OutT>
__global__ void lp_postnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, OutT* __restrict__ xc, int width,
                                   float alpha, float eps) {
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * width;
    OutT* cr = xc + (size_t)r * width;
    if (!w) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) cr[c] = from_f<OutT>(xr[c]);
        return;
    }
    const float* yr = y ? y + (size_t)r * width : nullptr;
    __shared__ float red[33];
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = yr ? fmaf(alpha, xr[c], yr[c]) : alpha * xr[c];
        xr[c] = v;
        ss += v * v;
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
    for (int c = threadIdx.x; c < width; c += blockDim.x) {   // (a thread reads back its own writes)
        const float v = xr[c] * inv * w[c];
        xr[c] = v;
        cr[c] = from_f<OutT>(v);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// out[r][n] = gelu_tanh(P[r][n]) * P[r][ff + n]: the fused projection holds [gate | up]
template <typename OutT>
__global__ void lp_gated_gelu_kernel(const float* __restrict__ P, int ldp, OutT* __restrict__ out, int ff, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * ff) return;
    const int r = (int)(i / ff), n = (int)(i - (size_t)r * ff);
    const float* p = P + (size_t)r * ldp;
    out[i] = from_f<OutT>(gelu_tanh_f(p[n]) * p[ff + n]);
}

// out[r][n] = relu(P[r][n])^2 (the relu^2 layer when its up projection is part of a wider product)
template <typename OutT>
__global__ void lp_relu2_kernel(const float* __restrict__ P, int ldp, OutT* __restrict__ out, int ff, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * ff) return;
    const int r = (int)(i / ff), n = (int)(i - (size_t)r * ff);
    const float z = fmaxf(P[(size_t)r * ldp + n], 0.0f);
    out[i] = from_f<OutT>(z * z);
}

// Router: one warp per row of the f32 logits P[r][0 .. E) (route_row, lp_rows_tail.cuh)
__global__ void lp_moe_route_kernel(const float* __restrict__ P, int ldp, int E, int top, float* __restrict__ wts, int* __restrict__ sel,
                                    float* __restrict__ selw, int R, int mode, float scale) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= R) return;
    route_row(P + (size_t)r * ldp, E, top, wts + (size_t)r * E, sel + (size_t)r * top, selw + (size_t)r * top, lane, mode, scale);
}

// an expert's activation: relu(z)^2 (B200_ACT_RELU2) or the exact GELU (B200_ACT_GELU)
__device__ __forceinline__ float expert_act(float z, int act) {
    if (act == B200_ACT_GELU) return gelu_erf_f(z);
    z = fmaxf(z, 0.0f);
    return z * z;
}

// A gated expert (B200_ACT_SILU_GLU) has two pre-activations per hidden unit, silu(g) * u; its up matrix is [gate | up] rows.
__device__ __forceinline__ int expert_rows(int eff, int act) { return act == B200_ACT_SILU_GLU ? 2 * eff : eff; }
// hidden unit of an expert from its pre-activation(s) and the expert's weight w: on the output, act(.) w, or on the input (win),
// where W (w h) = w (W h) puts it on the pre-activations
__device__ __forceinline__ float expert_unit(float z, float zu, float w, int act, int win) {
    if (win) { z *= w; zu *= w; }
    const float v = act == B200_ACT_SILU_GLU ? z * sigmoid_f(z) * zu : expert_act(z, act);
    return win ? v : v * w;
}

// out[r][c] = hidden unit c of the row: expert e = c / eff with its weight (0 = not chosen: the unit is 0), the always-on expert's
// units behind them with weight 1.  P holds every expert's pre-activations side by side (expert_rows per expert).
template <typename OutT>
__global__ void lp_moe_act_kernel(const float* __restrict__ P, int ldp, int off, const float* __restrict__ wts, int E, int eff, int total,
                                  OutT* __restrict__ out, int R, int act, int win) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * total) return;
    const int r = (int)(i / total), c = (int)(i - (size_t)r * total);
    const int e = c / eff, per = expert_rows(eff, act);
    const float wgt = e < E ? wts[(size_t)r * E + e] : 1.0f;
    float v = 0.0f;
    if (wgt != 0.0f) {
        const float* p = P + (size_t)r * ldp + off;
        if (e < E) v = expert_unit(p[e * per + (c - e * eff)], act == B200_ACT_SILU_GLU ? p[e * per + eff + (c - e * eff)] : 0.0f, wgt, act, win);
        else v = expert_act(p[E * per + (c - E * eff)], act);
    }
    out[i] = from_f<OutT>(v);
}

// The same for (token, choice) pairs in expert order: pair i = (row i / top, choice i % top) sits at row pos[i] of P (its expert's
// pre-activations, expert_rows wide) and of out (eff wide); its weight is selw[i].
template <typename OutT>
__global__ void lp_moe_pair_act_kernel(const float* __restrict__ P, int ldp, const int* __restrict__ pos, const float* __restrict__ selw, int eff,
                                       OutT* __restrict__ out, int n_pairs, int act, int win) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_pairs * eff) return;
    const int pr = (int)(i / eff), n = (int)(i - (size_t)pr * eff);
    const float* p = P + (size_t)pos[pr] * ldp;
    out[(size_t)pos[pr] * eff + n] = from_f<OutT>(expert_unit(p[n], act == B200_ACT_SILU_GLU ? p[eff + n] : 0.0f, selw[pr], act, win));
}

// Few rows (decoding): only the chosen experts' weights are read.  up_exp holds [e0 up | e1 up | ... | always-on up] rows of `width`
// columns (a gated expert: [gate | up], expert_rows each); segment k < top of a row's activations belongs to expert sel[r][k],
// segment `top` to the always-on expert.
//   act[r][k eff + n] = unit(up_e[n] . h_r, selw[r][k])        act[r][top eff + n] = act(up_shared[n] . h_r)      (expert_unit)
// One warp per (row, segment, n); h rows are staged in shared memory once per block.
template <typename T>
__global__ void __launch_bounds__(256) lp_moe_up_sel_kernel(const T* __restrict__ H, const T* __restrict__ up_exp, const int* __restrict__ sel,
                                                            const float* __restrict__ selw, int E, int top, int eff, int sff, int width, int R,
                                                            T* __restrict__ act, int act_kind, int win) {
    extern __shared__ __align__(16) uint8_t mu_smem[];
    T* hs = reinterpret_cast<T*>(mu_smem);
    constexpr int VN = Vec8<T>::N;
    for (int i = threadIdx.x; i < R * width / VN; i += blockDim.x)
        *reinterpret_cast<uint4*>(hs + (size_t)i * VN) = *reinterpret_cast<const uint4*>(H + (size_t)i * VN);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int per_row = top * eff + sff;
    const int total = R * per_row;
    for (int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); o < total; o += gridDim.x * (blockDim.x >> 5)) {
        const int r = o / per_row, c = o - r * per_row;
        const int k = c < top * eff ? c / eff : top;
        const int n = c - k * eff;
        const int e = k < top ? sel[(size_t)r * top + k] : E;
        const int per = expert_rows(eff, act_kind);
        const bool glu = act_kind == B200_ACT_SILU_GLU && k < top;
        const T* wr = up_exp + ((size_t)e * per + n) * width;
        const T* wu = wr + (size_t)eff * width;          // (gated experts: the up row of the same unit)
        const T* hr = hs + (size_t)r * width;
        float acc = 0.0f, accu = 0.0f;
        for (int i = lane * VN; i < width; i += 32 * VN) {
            float wv[VN], xv[VN];
            Vec8<T>::load(wr + i, wv);
            Vec8<T>::load(hr + i, xv);
#pragma unroll
            for (int j = 0; j < VN; j++) acc = fmaf(wv[j], xv[j], acc);
            if (glu) {
                Vec8<T>::load(wu + i, wv);
#pragma unroll
                for (int j = 0; j < VN; j++) accu = fmaf(wv[j], xv[j], accu);
            }
        }
        acc = wsum(acc);
        accu = wsum(accu);
        if (lane == 0) act[o] = from_f<T>(k < top ? expert_unit(acc, accu, selw[(size_t)r * top + k], act_kind, win) : expert_act(acc, act_kind));
    }
}

// y[r][c] = sum over the row's segments of down_e[c] . act segment; down_cat is [width][E eff + sff].  MD_SPLIT warps share one (row, c):
// each takes every MD_SPLIT-th 16-byte group of every segment (more loads in flight per output: a decode step has only `width` of
// them), the partial sums meet in shared memory and are added in warp order.  accum = 1: y += (y is the residual stream).
constexpr int MD_SPLIT = 4;
template <typename T>
__global__ void __launch_bounds__(256) lp_moe_down_sel_kernel(const T* __restrict__ act, const T* __restrict__ down_cat, const int* __restrict__ sel,
                                                              int E, int top, int eff, int sff, int width, int R, float* __restrict__ y, RowsTail tail, int accum) {
    constexpr int VN = Vec8<T>::N, GROUPS = 8 / MD_SPLIT;
    __shared__ float part[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = warp / MD_SPLIT, sw = warp % MD_SPLIT;
    const int per_row = top * eff + sff, kd = E * eff + sff, total = R * width;
    for (int base = blockIdx.x * GROUPS; base < total; base += gridDim.x * GROUPS) {
        const int o = base + grp;
        float acc = 0.0f;
        if (o < total) {
            const int r = o / width, c = o - r * width;
            const T* ar = act + (size_t)r * per_row;
            const T* dr = down_cat + (size_t)c * kd;
            for (int k = 0; k <= top; k++) {
                const int e = k < top ? sel[(size_t)r * top + k] : E;
                const int len = k < top ? eff : sff;
                const T* w = dr + (size_t)e * eff;
                const T* a = ar + (size_t)k * eff;
#pragma unroll 4
                for (int i = (sw * 32 + lane) * VN; i < len; i += MD_SPLIT * 32 * VN) {
                    float wv[VN], xv[VN];
                    Vec8<T>::load(w + i, wv);
                    Vec8<T>::load(a + i, xv);
#pragma unroll
                    for (int j = 0; j < VN; j++) acc = fmaf(wv[j], xv[j], acc);
                }
            }
        }
        acc = wsum(acc);
        if (lane == 0) part[warp] = acc;
        __syncthreads();
        if (o < total && sw == 0 && lane == 0) {
            float t = part[grp * MD_SPLIT];
#pragma unroll
            for (int i = 1; i < MD_SPLIT; i++) t += part[grp * MD_SPLIT + i];
            y[o] = accum ? y[o] + t : t;
        }
        __syncthreads();
    }
    if (tail.on) rows_tail<T>(tail);
}

// Many rows: the (token, choice) pairs are put in expert order, so that every expert multiplies a contiguous block of rows.
// One block: counts per expert, their running sum (seg[e] = {first row, rows}), then every pair takes the next free row of its
// expert (pos[r top + k]).  Which pair of an expert gets which row does not matter: a row's result does not depend on its place.
__global__ void __launch_bounds__(1024) lp_moe_sort_kernel(const int* __restrict__ sel, int n_pairs, int E, int* __restrict__ seg, int* __restrict__ pos) {
    extern __shared__ int ms[];          // [E] counts, then [E] cursors
    int* cnt = ms;
    int* cur = ms + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[sel[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; e++) {
            seg[2 * e] = at;
            seg[2 * e + 1] = cnt[e];
            cur[e] = at;
            at += cnt[e];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) pos[i] = atomicAdd(&cur[sel[i]], 1);
}

// Xp[pos[i]] = H[i / top]: one block per pair
template <typename T>
__global__ void lp_moe_gather_kernel(const T* __restrict__ H, const int* __restrict__ pos, int top, int width, T* __restrict__ Xp) {
    const int i = blockIdx.x;
    const T* src = H + (size_t)(i / top) * width;
    T* dst = Xp + (size_t)pos[i] * width;
    constexpr int VN = Vec8<T>::N;
    if (width % VN == 0) {
        for (int c = threadIdx.x; c < width / VN; c += blockDim.x) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
    }
}

// y[r] (+)= sum_k selw[r][k] Yp[pos[r top + k]], choices in the order they were taken; add = 1 when y already holds something to add
// to (the always-on expert's output, or the residual stream); selw = null: plain sum (the weights went into the experts' inputs)
__global__ void lp_moe_combine_kernel(const float* __restrict__ Yp, const int* __restrict__ pos, const float* __restrict__ selw, int top, int width,
                                      int add, float* __restrict__ y) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = add ? y[(size_t)r * width + c] : 0.0f, sum = 0.0f;
        for (int k = 0; k < top; k++) sum = fmaf(selw ? selw[(size_t)r * top + k] : 1.0f, Yp[(size_t)pos[(size_t)r * top + k] * width + c], sum);
        y[(size_t)r * width + c] = acc + sum;
    }
}

__global__ void lp_add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}
