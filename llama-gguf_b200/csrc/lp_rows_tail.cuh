// lp_rows_tail.cuh — what the LAST block of a few-row kernel (decoding) does once every block has written its part of a sublayer's
// output y: the norm after the residual sum, x <- (alpha x + y) / rms * w with the copy in the compute type, and, when a mixture of
// experts comes next, the router's logits on that copy and the choice of experts.  It replaces two to three launches of a few
// microseconds each per sublayer.  Included by layerprog.cu inside its anonymous namespace (after Vec8).
#pragma once

// Router of a mixture of experts for one row, by one warp: the `top` largest of z[0 .. E) are taken one after the other (of equal
// logits the lower index first); their weights are the softmax over the chosen logits only (mode B200_ROUTE_TOP_SOFTMAX), or their
// share of the softmax over ALL experts times `scale`, not renormalised (B200_ROUTE_SOFTMAX_TOP).  w[e] receives the weight of
// expert e (0 when it is not chosen); sel[k] / selw[k] list the chosen experts in the order they were taken.
__device__ __forceinline__ void route_row(const float* __restrict__ z, int E, int top, float* __restrict__ w, int* __restrict__ sel,
                                          float* __restrict__ selw, int lane, int mode, float scale) {
    for (int e = lane; e < E; e += 32) w[e] = 0.0f;
    __syncwarp();
    float zmax = 0.0f, sum = 0.0f;
    float all = 0.0f;
    if (mode == B200_ROUTE_SOFTMAX_TOP) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = wmax(mx);
        for (int e = lane; e < E; e += 32) all += expf(z[e] - mx);
        all = wsum(all);
    }
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (w[e] == 0.0f && (v > best || (v == best && e < bi))) { best = v; bi = e; }   // (chosen experts carry a mark != 0)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == 0) {
            w[bi] = -1.0f - p;          // mark; turned into the weight below
            sel[k] = bi;
            selw[k] = p;
        }
        __syncwarp();
    }
    const float inv = mode == B200_ROUTE_SOFTMAX_TOP ? scale / all : 1.0f / sum;
    for (int e = lane; e < E; e += 32)
        if (w[e] != 0.0f) w[e] = (-1.0f - w[e]) * inv;
    for (int k = lane; k < top; k += 32) selw[k] *= inv;
    __syncwarp();
}

struct RowsTail {
    int on;                             // 0: the kernel ends as usual
    float* x;                           // [R][width] residual stream, f32
    const float* y;                     // [R][width] what the kernel's blocks have written
    const float* w;                     // norm weight
    void* xc;                           // [R][width] copy in the compute type
    int width, R;
    float alpha, eps;
    unsigned* counter;                  // zero before the launch; the last block sets it back
    const void* router;                 // [E][width] in the compute type, or null
    int E, top;
    int route;                          // B200_ROUTE_*
    float route_scale;
    float *logits, *wts, *selw;         // [R][E], [R][E], [R][top]
    int* sel;                           // [R][top]
};

// Called by every thread of every block after the block's own stores.  Returns after the tail's work in the last block.
// The norm: nw / wpr rows at a time, wpr warps per row (all eight for one row, one per row from eight rows on).  A thread loads its
// elements eight at a time before it stores any of them (a store between two loads would make every load wait for the one before).
template <typename T>
__device__ void rows_tail(const RowsTail& t) {
    __shared__ int is_last;
    __shared__ float part[8];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(t.counter, 1u) == gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;   // (blockDim.x = 256)
    T* xc = reinterpret_cast<T*>(t.xc);
    int wpr = nw;
    while (wpr > 1 && nw / wpr < t.R) wpr >>= 1;
    const int rows_par = nw / wpr, grp = warp / wpr, tig = (warp % wpr) * 32 + lane, T_ = wpr * 32;
    for (int r0 = 0; r0 < t.R; r0 += rows_par) {
        const int r = r0 + grp;
        const bool live = r < t.R;
        float* xr = t.x + (size_t)(live ? r : 0) * t.width;
        const float* yr = t.y + (size_t)(live ? r : 0) * t.width;
        T* cr = xc + (size_t)(live ? r : 0) * t.width;
        float ss = 0.0f;
        if (live) {
            for (int c0 = tig; c0 < t.width; c0 += 8 * T_) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = c0 + j * T_;
                    v[j] = c < t.width ? fmaf(t.alpha, xr[c], __ldcg(yr + c)) : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = c0 + j * T_;
                    if (c < t.width) xr[c] = v[j];
                    ss += v[j] * v[j];
                }
            }
        }
        ss = wsum(ss);
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (int i = 0; i < wpr; i++) tot += part[grp * wpr + i];
        __syncthreads();
        if (live) {
            const float inv = 1.0f / sqrtf(tot / (float)t.width + t.eps);
            for (int c0 = tig; c0 < t.width; c0 += 8 * T_) {   // (a thread reads back its own writes)
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = c0 + j * T_;
                    v[j] = c < t.width ? xr[c] * inv * t.w[c] : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = c0 + j * T_;
                    if (c < t.width) {
                        xr[c] = v[j];
                        cr[c] = from_f<T>(v[j]);
                    }
                }
            }
        }
    }
    if (t.router) {
        __syncthreads();                                // the copies of all rows are in place (this block wrote them)
        const T* rw = reinterpret_cast<const T*>(t.router);
        constexpr int VN = Vec8<T>::N;
        const bool vec = t.width % VN == 0;
        for (int o = warp; o < t.R * t.E; o += nw) {    // a warp per (row, expert): the logit in f32
            const int r = o / t.E, e = o - r * t.E;
            const T* wr = rw + (size_t)e * t.width;
            const T* hr = xc + (size_t)r * t.width;
            float acc = 0.0f;
            if (vec) {
                for (int c = lane * VN; c < t.width; c += 32 * VN) {
                    float wv[VN], xv[VN];
                    Vec8<T>::load(wr + c, wv);
                    Vec8<T>::load(hr + c, xv);
#pragma unroll
                    for (int j = 0; j < VN; j++) acc = fmaf(wv[j], xv[j], acc);
                }
            } else {
                for (int c = lane; c < t.width; c += 32) acc = fmaf(to_f(wr[c]), to_f(hr[c]), acc);
            }
            acc = wsum(acc);
            if (lane == 0) t.logits[(size_t)r * t.E + e] = acc;
        }
        __syncthreads();
        for (int r = warp; r < t.R; r += nw)
            route_row(t.logits + (size_t)r * t.E, t.E, t.top, t.wts + (size_t)r * t.E, t.sel + (size_t)r * t.top, t.selw + (size_t)r * t.top, lane, t.route, t.route_scale);
    }
    if (threadIdx.x == 0) *t.counter = 0u;
}
