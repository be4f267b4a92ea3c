// lp_latent_attn.cuh — what the latent-attention mixer (B200_MIX_LATENT_ATTN) does around the library's GEMMs and attention kernels.
// The cache of a layer run holds one row per position, [c (kv_rank) | rotated shared key part (rot_dim)], f32; the attention kernels
// of layerprog.cu read it as ONE K/V head whose keys are the whole row and whose values are the row's first kv_rank entries
// (AttnGeom.v_in_k).  For that, head n's query is carried into the latent: qbuf[r][n] = [W_uk[n]^T q_plain | rotated q part], and the
// summed latent comes back through W_uv[n] afterwards (two products batched over the heads).  Included by layerprog.cu inside its
// anonymous namespace.  Norms, angles and the rotation are f32 (the angle, its sine and cosine in double).
#pragma once

struct LatentGeom {
    int H, dim, rot_dim, vdim, q_rank, kv_rank;
    int rot_n;               // rotated channels (even, <= rot_dim); channel i pairs with i + rot_n / 2
    float rot_mult;          // factor on cos and sin
    int q_off, kv_off, g_off;   // columns of the fused input projection P: [W_dq h | W_dkv h | W_g h]; kv_off < 0: no W_dkv (borrowed rows)
    size_t cache_off;        // byte offset of the rows inside a slot's cache block
    int cap;
    float eps;
};

// cos / sin of the row's position into shared memory: cs[i], sn[i], i < rot_n / 2
__device__ __forceinline__ void latent_angles(const LatentGeom& g, const double* __restrict__ freq, int pos, float* cs, float* sn) {
    for (int i = threadIdx.x; i < g.rot_n / 2; i += blockDim.x) {
        double s, c;
        sincos((double)pos * freq[i], &s, &c);
        cs[i] = (float)c * g.rot_mult;
        sn[i] = (float)s * g.rot_mult;
    }
}
__device__ __forceinline__ float latent_rot(const LatentGeom& g, const float* v, int i, const float* cs, const float* sn) {
    const int half = g.rot_n / 2;
    if (i >= g.rot_n) return v[i];
    return i < half ? v[i] * cs[i] - v[i + half] * sn[i] : v[i] * cs[i - half] + v[i - half] * sn[i - half];
}

// One block per row, after the fused input projection.  c_q = rmsnorm(P[q_off ..]) * qw -> cq (compute type, the operand of W_uq).
// With a W_dkv of its own: c = rmsnorm(P[kv_off .. + kv_rank]) * kvw and the rotated last rot_dim columns -> the cache row of the
// row's position.
template <typename T>
__global__ void __launch_bounds__(256) lp_latent_prep_kernel(StepMeta sm, LatentGeom g, const float* __restrict__ P, int ldp,
                                                             const float* __restrict__ qw, const float* __restrict__ kvw,
                                                             const double* __restrict__ freq, T* __restrict__ cq) {
    extern __shared__ float lp_cs[];     // [rot_n / 2] cos, then sin
    __shared__ float red[2][8];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int run = sm.row_run[r], pos = sm.row_pos[r];
    const float* p = P + (size_t)r * ldp;
    float* cs = lp_cs;
    float* sn = lp_cs + g.rot_n / 2;
    const bool own = g.kv_off >= 0;
    if (own) latent_angles(g, freq, pos, cs, sn);
    float sq = 0.0f, sk = 0.0f;
    for (int c = threadIdx.x; c < g.q_rank; c += blockDim.x) sq = fmaf(p[g.q_off + c], p[g.q_off + c], sq);
    if (own)
        for (int c = threadIdx.x; c < g.kv_rank; c += blockDim.x) sk = fmaf(p[g.kv_off + c], p[g.kv_off + c], sk);
    sq = wsum(sq);
    sk = wsum(sk);
    if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    __syncthreads();
    sq = 0.0f; sk = 0.0f;
    for (int i = 0; i < nw; i++) { sq += red[0][i]; sk += red[1][i]; }
    const float iq = 1.0f / sqrtf(sq / (float)g.q_rank + g.eps);
    for (int c = threadIdx.x; c < g.q_rank; c += blockDim.x) cq[(size_t)r * g.q_rank + c] = from_f<T>(p[g.q_off + c] * iq * qw[c]);
    if (!own) return;
    const float ik = 1.0f / sqrtf(sk / (float)g.kv_rank + g.eps);
    float* row = reinterpret_cast<float*>(sm.run_kv[run] + g.cache_off) + (size_t)pos * (g.kv_rank + g.rot_dim);
    for (int c = threadIdx.x; c < g.kv_rank; c += blockDim.x) row[c] = p[g.kv_off + c] * ik * kvw[c];
    const float* kr = p + g.kv_off + g.kv_rank;
    for (int i = threadIdx.x; i < g.rot_dim; i += blockDim.x) row[g.kv_rank + i] = latent_rot(g, kr, i, cs, sn);
}

// One block per row, after q = W_uq c_q (Q [R][H (dim + rot_dim)] f32): the plain part of every head in the compute type -> qn
// [R][H dim] (the operand of the product with W_uk^T), the rotated part -> qbuf[r][n (kv_rank + rot_dim) + kv_rank ..].
template <typename T>
__global__ void __launch_bounds__(256) lp_latent_qprep_kernel(StepMeta sm, LatentGeom g, const float* __restrict__ Q, const double* __restrict__ freq,
                                                              T* __restrict__ qn, float* __restrict__ qbuf) {
    extern __shared__ float lq_cs[];
    const int r = blockIdx.x, pos = sm.row_pos[r];
    float* cs = lq_cs;
    float* sn = lq_cs + g.rot_n / 2;
    latent_angles(g, freq, pos, cs, sn);
    __syncthreads();
    const int per = g.dim + g.rot_dim, D = g.kv_rank + g.rot_dim;
    const float* q = Q + (size_t)r * g.H * per;
    for (int i = threadIdx.x; i < g.H * per; i += blockDim.x) {
        const int n = i / per, c = i - n * per;
        if (c < g.dim) qn[(size_t)r * g.H * g.dim + n * g.dim + c] = from_f<T>(q[i]);
        else qbuf[(size_t)r * g.H * D + (size_t)n * D + g.kv_rank + (c - g.dim)] = latent_rot(g, q + n * per + g.dim, c - g.dim, cs, sn);
    }
}

// out[r][c] = V[r][c] * sigmoid(P[r][g_off + c]) in the compute type (gate = 0: a plain conversion): the operand of W_o
template <typename T>
__global__ void lp_latent_gate_kernel(const float* __restrict__ V, const float* __restrict__ P, int ldp, int g_off, int gate, int n, int R,
                                      T* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * n) return;
    const int r = (int)(i / n), c = (int)(i - (size_t)r * n);
    const float v = V[i];
    out[i] = from_f<T>(gate ? v * sigmoid_f(P[(size_t)r * ldp + g_off + c]) : v);
}
