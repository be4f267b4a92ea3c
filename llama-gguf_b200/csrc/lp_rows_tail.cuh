// lp_rows_tail.cuh — what the LAST block of a few-row kernel (decoding) does once every block has written its part of a sublayer's
// output y: the norm after the residual sum, x <- (alpha x + y) / rms * w with the copy in the compute type, and, when a mixture of
// experts comes next, the router's logits on that copy and the choice of experts.  It replaces two to three launches of a few
// microseconds each per sublayer.  Included by layerprog.cu inside its anonymous namespace (after Vec8).
#pragma once

// Router of a mixture of experts for one row, by one warp: the `top` largest of z[0 .. E) are taken one after the other (of equal
// logits the lower index first); their weights are the softmax over the chosen logits only (mode B200_ROUTE_TOP_SOFTMAX), or their
// share of the softmax over ALL experts times `scale`, not renormalised (B200_ROUTE_SOFTMAX_TOP), or their own sigmoid, not
// renormalised, times `scale` when that is not 0 (B200_ROUTE_SIGMOID_TOP).  w[e] receives the weight of
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
        const float p = mode == B200_ROUTE_SIGMOID_TOP ? sigmoid_f(best) : expf(best - zmax);
        sum += p;
        if (lane == 0) {
            w[bi] = -1.0f - p;          // mark; turned into the weight below
            sel[k] = bi;
            selw[k] = p;
        }
        __syncwarp();
    }
    const float inv = mode == B200_ROUTE_SIGMOID_TOP ? (scale != 0.0f ? scale : 1.0f) : mode == B200_ROUTE_SOFTMAX_TOP ? scale / all : 1.0f / sum;
    for (int e = lane; e < E; e += 32)
        if (w[e] != 0.0f) w[e] = (-1.0f - w[e]) * inv;
    for (int k = lane; k < top; k += 32) selw[k] *= inv;
    __syncwarp();
}

// What the multi-stream layer form does between two sublayers (lp_streams.cuh has the kernel for many rows; rows_tail below does
// the same for few rows inside the kernel that wrote y).
constexpr int ST_MAX = 8;   // streams at most (they live in registers)
struct StreamStep {
    int S, width;
    const float* src;        // [R][width]: every stream starts as this row (the embedding); null: the streams hold their values
    const float* y;          // [R][width] output of the sublayer before, or null
    const float* mix;        // [S][S] (from, to) of that sublayer, null = identity
    const float* out;        // [S], null = ones
    float mult;              // factor on y
    const float* in;         // [S] weights of the next sublayer's input, null = ones (the plain sum)
    const float* w;          // norm weight of the next sublayer, null = no norm and no compute-type copy
    int center;              // 1: layer norm (mean taken off), 0: RMS norm
    float eps;
    float* sum;              // [R][width]: receives the plain sum of the streams, or null
};

struct RowsTail {
    int on;                             // 0: the kernel ends as usual
    int streams;                        // 1: the multi-stream form: `st` says what to do with y, xs holds the copies [R][S][width]
    StreamStep st;
    float* xs;
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
    if (t.streams) {
        // Row by row, the whole block: the copies are updated from y (pass 1, which also sums the next input u), then u is formed
        // twice more from the copies this thread has just written (no row buffer: the kernel's shared memory belongs to its main
        // part) for the variance and for the normed row.
        const StreamStep& st = t.st;
        const int S = st.S, W = st.width;
        __shared__ float mix_s[ST_MAX * ST_MAX], out_s[ST_MAX], in_s[ST_MAX];
        __shared__ float tot_s;
        if (threadIdx.x < S * S) mix_s[threadIdx.x] = st.mix ? st.mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.0f : 0.0f);
        if (threadIdx.x < S) {
            out_s[threadIdx.x] = (st.out ? st.out[threadIdx.x] : 1.0f) * st.mult;
            in_s[threadIdx.x] = st.in ? st.in[threadIdx.x] : 1.0f;
        }
        __syncthreads();
        auto block_sum = [&](float v) {
            v = wsum(v);
            __syncthreads();
            if (lane == 0) part[warp] = v;
            __syncthreads();
            if (threadIdx.x == 0) {
                float a = 0.0f;
                for (int i = 0; i < nw; i++) a += part[i];
                tot_s = a;
            }
            __syncthreads();
            return tot_s;
        };
        // Rows up to 4096 wide (a multiple of 4): a thread owns up to TG groups of 4 channels; all their loads are issued before the
        // first store, and the next input u stays in registers for the variance and the normed row.
        constexpr int TG = 4;
        const bool fast = (W & 3) == 0 && W <= 4 * 256 * TG && S <= 4;
        for (int r = 0; r < (fast ? t.R : 0); r++) {
            float* xr = t.xs + (size_t)r * S * W;
            const float* yr = st.y + (size_t)r * W;
            float4 v[TG][4], yv[TG];
            float u[TG][4];
#pragma unroll
            for (int g = 0; g < TG; g++) {
                const int c = (threadIdx.x + g * 256) * 4;
                if (c < W) {
                    yv[g] = __ldcg(reinterpret_cast<const float4*>(yr + c));
#pragma unroll
                    for (int s = 0; s < 4; s++)
                        v[g][s] = s < S ? *reinterpret_cast<const float4*>(xr + (size_t)s * W + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float tot = 0.0f;
#pragma unroll
            for (int g = 0; g < TG; g++) {
                const int c = (threadIdx.x + g * 256) * 4;
                u[g][0] = u[g][1] = u[g][2] = u[g][3] = 0.0f;
                if (c < W) {
                    const float y4[4] = {yv[g].x, yv[g].y, yv[g].z, yv[g].w};
                    float o4[4][4], plain[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int s = 0; s < 4; s++) {
                            if (s < S && k < S) {
                                const float mx = mix_s[s * S + k];
                                a[0] = fmaf(mx, v[g][s].x, a[0]);
                                a[1] = fmaf(mx, v[g][s].y, a[1]);
                                a[2] = fmaf(mx, v[g][s].z, a[2]);
                                a[3] = fmaf(mx, v[g][s].w, a[3]);
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 4; e++) o4[k][e] = k < S ? fmaf(out_s[k], y4[e], a[e]) : 0.0f;
                    }
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        if (k < S) {
                            *reinterpret_cast<float4*>(xr + (size_t)k * W + c) = make_float4(o4[k][0], o4[k][1], o4[k][2], o4[k][3]);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                u[g][e] = fmaf(in_s[k], o4[k][e], u[g][e]);
                                plain[e] += o4[k][e];
                            }
                        }
                    }
                    if (st.sum) *reinterpret_cast<float4*>(st.sum + (size_t)r * W + c) = make_float4(plain[0], plain[1], plain[2], plain[3]);
                    tot += (u[g][0] + u[g][1]) + (u[g][2] + u[g][3]);
                }
            }
            if (!st.w) continue;
            const float mean = st.center ? block_sum(tot) / (float)W : 0.0f;
            float sq = 0.0f;
#pragma unroll
            for (int g = 0; g < TG; g++)
                if ((threadIdx.x + g * 256) * 4 < W)
#pragma unroll
                    for (int e = 0; e < 4; e++) sq = fmaf(u[g][e] - mean, u[g][e] - mean, sq);
            const float inv = 1.0f / sqrtf(block_sum(sq) / (float)W + st.eps);
#pragma unroll
            for (int g = 0; g < TG; g++) {
                const int c = (threadIdx.x + g * 256) * 4;
                if (c < W) {
                    const float4 wv = *reinterpret_cast<const float4*>(st.w + c);
                    const float w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) xc[(size_t)r * W + c + e] = from_f<T>((u[g][e] - mean) * inv * w4[e]);
                }
            }
        }
        for (int r = 0; r < (fast ? 0 : t.R); r++) {
            float* xr = t.xs + (size_t)r * S * W;
            const float* yr = st.y + (size_t)r * W;
            float tot = 0.0f;
            for (int c = threadIdx.x; c < W; c += blockDim.x) {
                float v[ST_MAX], nv[ST_MAX];
#pragma unroll
                for (int s = 0; s < ST_MAX; s++) v[s] = s < S ? xr[(size_t)s * W + c] : 0.0f;
                const float yv = __ldcg(yr + c);
                float u = 0.0f, plain = 0.0f;
#pragma unroll
                for (int k = 0; k < ST_MAX; k++) {
                    float a = 0.0f;
#pragma unroll
                    for (int s = 0; s < ST_MAX; s++)
                        if (s < S && k < S) a = fmaf(mix_s[s * S + k], v[s], a);
                    nv[k] = k < S ? fmaf(out_s[k], yv, a) : 0.0f;
                }
#pragma unroll
                for (int s = 0; s < ST_MAX; s++) {
                    if (s < S) {
                        xr[(size_t)s * W + c] = nv[s];
                        u = fmaf(in_s[s], nv[s], u);
                        plain += nv[s];
                    }
                }
                if (st.sum) st.sum[(size_t)r * W + c] = plain;
                tot += u;
            }
            if (!st.w) continue;
            auto u_of = [&](int c) {
                float u = 0.0f;
#pragma unroll
                for (int s = 0; s < ST_MAX; s++)
                    if (s < S) u = fmaf(in_s[s], xr[(size_t)s * W + c], u);
                return u;
            };
            const float mean = st.center ? block_sum(tot) / (float)W : 0.0f;
            float sq = 0.0f;
            for (int c = threadIdx.x; c < W; c += blockDim.x) {   // (a thread reads back its own writes)
                const float d = u_of(c) - mean;
                sq = fmaf(d, d, sq);
            }
            const float inv = 1.0f / sqrtf(block_sum(sq) / (float)W + st.eps);
            for (int c = threadIdx.x; c < W; c += blockDim.x) xc[(size_t)r * W + c] = from_f<T>((u_of(c) - mean) * inv * st.w[c]);
        }
    }
    int wpr = nw;
    while (wpr > 1 && nw / wpr < t.R) wpr >>= 1;
    const int rows_par = nw / wpr, grp = warp / wpr, tig = (warp % wpr) * 32 + lane, T_ = wpr * 32;
    for (int r0 = 0; r0 < (t.streams ? 0 : t.R); r0 += rows_par) {
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
    if (t.router && (!t.streams || t.st.w)) {
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
