// lp_streams.cuh — the multi-stream layer form (program.streams >= 1): the residual is S copies of the embedding; a sublayer reads a
// weighted sum of them through a norm, and its output y updates all copies at once through an S x S mixing matrix.  One kernel does
// what lies between two sublayers: the update after the one, the sum and the norm before the other.  Included by layerprog.cu
// inside its anonymous namespace.  Everything is f32; the normed row is rounded once to the compute type.
#pragma once

// (StreamStep: lp_rows_tail.cuh)

// One block per row.  xs [R][S][width].  Pass 1, per group of VEC channels (VEC = 4: 16-byte loads and stores, the width a multiple of
// 4): the S old values -> the S new ones (all loads of a group before its stores), their weighted sum u into shared memory.  Pass 2:
// mean and variance of u over the row (two passes over shared memory: the variance is the mean of the squared deviations),
// hn = (u - mean) / sqrt(var + eps) * w.
template <int VEC>
__device__ __forceinline__ void st_load(const float* p, float* o) {
    if (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else o[0] = *p;
}
template <int VEC>
__device__ __forceinline__ void st_store(float* p, const float* o) {
    if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    else *p = o[0];
}
// (SMAX: compile-time bound of the stream count, 4 or ST_MAX, so that few streams cost few registers)
template <typename OutT, int VEC, int SMAX>
__global__ void __launch_bounds__(256) lp_streams_kernel(float* __restrict__ xs, StreamStep st, OutT* __restrict__ hn) {
    extern __shared__ __align__(16) float u_s[];      // [width]
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
    const float* __restrict__ src = st.src ? st.src + (size_t)r * W : nullptr;
    const float* __restrict__ yr = st.y ? st.y + (size_t)r * W : nullptr;
    float* __restrict__ sum = st.sum ? st.sum + (size_t)r * W : nullptr;
    float tot = 0.0f;
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
        float v[SMAX][VEC], yv[VEC], nv[SMAX][VEC], u[VEC], plain[VEC];
        if (src) {
            st_load<VEC>(src + c, v[0]);
#pragma unroll
            for (int s = 1; s < SMAX; s++)
#pragma unroll
                for (int k = 0; k < VEC; k++) v[s][k] = v[0][k];
        } else {
#pragma unroll
            for (int s = 0; s < SMAX; s++) {
                if (s < S) st_load<VEC>(xr + (size_t)s * W + c, v[s]);
                else
#pragma unroll
                    for (int k = 0; k < VEC; k++) v[s][k] = 0.0f;
            }
        }
        if (yr) {
            st_load<VEC>(yr + c, yv);
#pragma unroll
            for (int t = 0; t < SMAX; t++) {
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    float a = 0.0f;
#pragma unroll
                    for (int s = 0; s < SMAX; s++)
                        if (s < S && t < S) a = fmaf(mix_s[s * S + t], v[s][k], a);
                    nv[t][k] = t < S ? fmaf(out_s[t], yv[k], a) : 0.0f;
                }
            }
#pragma unroll
            for (int t = 0; t < SMAX; t++)
#pragma unroll
                for (int k = 0; k < VEC; k++) v[t][k] = nv[t][k];
        }
#pragma unroll
        for (int k = 0; k < VEC; k++) u[k] = plain[k] = 0.0f;
#pragma unroll
        for (int s = 0; s < SMAX; s++) {
            if (s < S) {
                if (yr || src) st_store<VEC>(xr + (size_t)s * W + c, v[s]);
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    u[k] = fmaf(in_s[s], v[s][k], u[k]);
                    plain[k] += v[s][k];
                }
            }
        }
        if (sum) st_store<VEC>(sum + c, plain);
        st_store<VEC>(u_s + c, u);
#pragma unroll
        for (int k = 0; k < VEC; k++) tot += u[k];
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
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {   // (a thread reads back its own entries of u_s)
#pragma unroll
        for (int k = 0; k < VEC; k++) {
            const float d = u_s[c + k] - mean;
            sq = fmaf(d, d, sq);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(sq) / (float)W + st.eps);
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
        float wv[VEC];
        st_load<VEC>(st.w + c, wv);
#pragma unroll
        for (int k = 0; k < VEC; k++) hn[(size_t)r * W + c + k] = from_f<OutT>((u_s[c + k] - mean) * inv * wv[k]);
    }
}
