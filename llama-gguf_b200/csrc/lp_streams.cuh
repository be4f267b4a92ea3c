// lp_streams.cuh — the multi-stream layer form (program.streams >= 1): the residual is S copies of the embedding; a sublayer reads a
// weighted sum of them through a norm, and its output y updates all copies at once through an S x S mixing matrix.  One kernel does
// what lies between two sublayers: the update after the one, the sum and the norm before the other.  Included by layerprog.cu
// inside its anonymous namespace.  Everything is f32; the normed row is rounded once to the compute type.
#pragma once

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

// One block per row.  xs [R][S][width].  Pass 1, per channel: the S old values -> the S new ones (stored), their weighted sum u into
// shared memory.  Pass 2: mean and variance of u over the row (two passes over shared memory: the variance is the mean of the squared
// deviations), hn = (u - mean) / sqrt(var + eps) * w.
template <typename OutT>
__global__ void __launch_bounds__(256) lp_streams_kernel(float* __restrict__ xs, StreamStep st, OutT* __restrict__ hn) {
    extern __shared__ float u_s[];      // [width]
    __shared__ float red[9];
    __shared__ float mix_s[ST_MAX * ST_MAX], out_s[ST_MAX], in_s[ST_MAX];
    const int r = blockIdx.x, S = st.S, W = st.width, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (threadIdx.x < S * S) mix_s[threadIdx.x] = st.mix ? st.mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.0f : 0.0f);
    if (threadIdx.x < S) {
        out_s[threadIdx.x] = (st.out ? st.out[threadIdx.x] : 1.0f) * st.mult;
        in_s[threadIdx.x] = st.in ? st.in[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    float* xr = xs + (size_t)r * S * W;
    float tot = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v[ST_MAX];
        if (st.src) {
            const float e = st.src[(size_t)r * W + c];
#pragma unroll
            for (int s = 0; s < ST_MAX; s++) v[s] = e;
        } else {
#pragma unroll
            for (int s = 0; s < ST_MAX; s++) v[s] = s < S ? xr[(size_t)s * W + c] : 0.0f;
        }
        if (st.y) {
            const float yv = st.y[(size_t)r * W + c];
            float nv[ST_MAX];
#pragma unroll
            for (int t = 0; t < ST_MAX; t++) {
                float a = 0.0f;
#pragma unroll
                for (int s = 0; s < ST_MAX; s++)
                    if (s < S && t < S) a = fmaf(mix_s[s * S + t], v[s], a);
                nv[t] = t < S ? fmaf(out_s[t], yv, a) : 0.0f;
            }
#pragma unroll
            for (int t = 0; t < ST_MAX; t++) v[t] = nv[t];
        }
        float u = 0.0f, plain = 0.0f;
#pragma unroll
        for (int s = 0; s < ST_MAX; s++) {
            if (s < S) {
                if (st.y || st.src) xr[(size_t)s * W + c] = v[s];
                u = fmaf(in_s[s], v[s], u);
                plain += v[s];
            }
        }
        if (st.sum) st.sum[(size_t)r * W + c] = plain;
        u_s[c] = u;
        tot += u;
    }
    if (!st.w) return;
    auto block_sum = [&](float v) {
        v = wsum(v);
        __syncthreads();
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int i = 0; i < nw; i++) t += red[i];
            red[8] = t;
        }
        __syncthreads();
        return red[8];
    };
    const float mean = st.center ? block_sum(tot) / (float)W : 0.0f;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {   // (a thread reads back its own entries of u_s)
        const float d = u_s[c] - mean;
        sq = fmaf(d, d, sq);
    }
    const float inv = 1.0f / sqrtf(block_sum(sq) / (float)W + st.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) hn[(size_t)r * W + c] = from_f<OutT>((u_s[c] - mean) * inv * st.w[c]);
}
