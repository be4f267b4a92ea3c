// lp_state_space.cuh — the recurrence and the gated group norm of the state-space mixer (B200_MIX_STATE_SPACE).  Its short
// convolution is lp_conv_silu_kernel / lp_conv_tail_kernel of layerprog.cu (column offset and bias).  Included by layerprog.cu inside
// its anonymous namespace, after the scan helpers.  The step size, the decay, the state and the norm are f32 in both compute modes.
#pragma once

// Columns: P (fused input projection) = [z (H vdim) | x | B (G N) | C (G N) | dt (H)]; XBC (after convolution + SiLU) = [x | B | C].
// State block of a run: S [H][N][vdim] | tail [taps - 1][H vdim + 2 G N], f32.
struct SsdGeom {
    int H, G, N, vdim;
    int dt_off;              // column of dt in P
    size_t rec_off;
};

// Per (run, head), laid out like the other scans: thread = value channel j, its state column S[:, j] cut into 16-entry pieces over
// neighbouring lanes, tokens staged in chunks.  (8-entry pieces -- twice the warps, half the state each -- were measured: 4 % slower
// on prompts, 10 % slower at batch 32.)  dt = softplus(z_dt + dt_bias), a = exp(-exp(A_log) dt):
//   S <- a S + B (dt x)^T;   y = S^T C + D x      (the read-out sees this token's write)
template <int DMAX>
__global__ void __launch_bounds__(SCAN_BD) lp_ssd_scan_kernel(StepMeta sm, SsdGeom g, const float* __restrict__ XBC, int ldc, const float* __restrict__ P,
                                                              int ldp, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                              const float* __restrict__ Dskip, float* __restrict__ O, int ldo) {
    constexpr int DREG = SCAN_DREG, CH = ScanChunk<DMAX>::N, SPLIT = DMAX / DREG, COLS = SCAN_BD / SPLIT;
    __shared__ __align__(16) float cs_[CH][DMAX];
    __shared__ __align__(16) float bs_[CH][DMAX];
    __shared__ float xs_[CH][COLS], dt_s[CH], dec_s[CH];
    const int tid = threadIdx.x, col = tid / SPLIT, sub = tid % SPLIT;
    const int j = blockIdx.x * COLS + col, h = blockIdx.y, run = blockIdx.z;
    const int grp = h * g.G / g.H;
    const int r0 = sm.run_start[run], r1 = sm.run_start[run + 1];
    float* Sg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)h * g.N * g.vdim;
    const bool live = j < g.vdim;
    float s[DREG];
#pragma unroll
    for (int i = 0; i < DREG; i++) {
        const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);   // state row of register i
        s[i] = (live && d < g.N) ? Sg[(size_t)d * g.vdim + j] : 0.0f;
    }
    for (int i = tid; i < CH * DMAX; i += SCAN_BD) {   // the padding beyond N stays zero
        (&cs_[0][0])[i] = 0.0f;
        (&bs_[0][0])[i] = 0.0f;
    }
    const float rate = expf(A_log[h]), dtb = dt_bias[h], dskip = Dskip[h];
    const int inner = g.H * g.vdim, b_col = inner + grp * g.N, c_col = inner + g.G * g.N + grp * g.N;
    const int jc = blockIdx.x * COLS + (tid % COLS);
    const bool vec = ((g.N | ldc | b_col | c_col) & 3) == 0 && (reinterpret_cast<uintptr_t>(XBC) & 15) == 0;
    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();
        if (vec) {   // 16-byte copies: a token's B and C rows are N / 4 chunks each
            const int per = g.N >> 2;
            for (int i = tid; i < nt * per; i += SCAN_BD) {
                const int t = i / per, d = (i - t * per) * 4;
                const float* x = XBC + (size_t)(c0 + t) * ldc;
                cp_async16(smem_u32(&bs_[t][d]), x + b_col + d, 16u);
                cp_async16(smem_u32(&cs_[t][d]), x + c_col + d, 16u);
            }
        } else {
            for (int t = 0; t < nt; t++) {
                const float* x = XBC + (size_t)(c0 + t) * ldc;
                for (int d = tid; d < g.N; d += SCAN_BD) {
                    cp_async4(&bs_[t][d], x + b_col + d);
                    cp_async4(&cs_[t][d], x + c_col + d);
                }
            }
        }
        for (int t = tid / COLS; t < nt; t += SPLIT) {
            if (jc < g.vdim) cp_async4(&xs_[t][tid % COLS], XBC + (size_t)(c0 + t) * ldc + h * g.vdim + jc);
            else xs_[t][tid % COLS] = 0.0f;
        }
        if (tid < nt) {
            const float dt = softplus_f(P[(size_t)(c0 + tid) * ldp + g.dt_off + h] + dtb);
            dt_s[tid] = dt;
            dec_s[tid] = expf(-rate * dt);
        }
        cp_async_wait_all();
        __syncthreads();
#pragma unroll 4
        for (int t = 0; t < nt; t++) {   // (unrolled: only the state's one multiply-add per token is serial, the read-outs overlap)
            const float decay = dec_s[t], x = xs_[t][col], dx = dt_s[t] * x;
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int i = 0; i < DREG; i += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(&bs_[t][((i >> 2) * SPLIT + sub) * 4]);
                const float4 c4 = *reinterpret_cast<const float4*>(&cs_[t][((i >> 2) * SPLIT + sub) * 4]);
                s[i] = fmaf(decay, s[i], b4.x * dx);
                s[i + 1] = fmaf(decay, s[i + 1], b4.y * dx);
                s[i + 2] = fmaf(decay, s[i + 2], b4.z * dx);
                s[i + 3] = fmaf(decay, s[i + 3], b4.w * dx);
                a0 = fmaf(s[i], c4.x, a0);
                a1 = fmaf(s[i + 1], c4.y, a1);
                a2 = fmaf(s[i + 2], c4.z, a2);
                a3 = fmaf(s[i + 3], c4.w, a3);
            }
            const float acc = split_sum<SPLIT>((a0 + a1) + (a2 + a3));
            if (live && sub == 0) O[(size_t)(c0 + t) * ldo + h * g.vdim + j] = fmaf(dskip, x, acc);
        }
    }
    if (live)
#pragma unroll
        for (int i = 0; i < DREG; i++) {
            const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);
            if (d < g.N) Sg[(size_t)d * g.vdim + j] = s[i];
        }
}

// out[r][c] = v / sqrt(mean over c's group of v^2 + eps) * w[c], v = O[r][c] * silu(P[r][z_off + c]); the row is cut into `groups` equal
// parts.  One block per (row, group).  The gate comes before the norm.
template <typename OutT>
__global__ void __launch_bounds__(256) lp_gate_groupnorm_kernel(const float* __restrict__ O, int ldo, const float* __restrict__ P, int ldp, int z_off,
                                                                const float* __restrict__ w, int n, int groups, float eps, OutT* __restrict__ out) {
    __shared__ float red[9];
    const int r = blockIdx.x, gi = blockIdx.y, len = n / groups, c0 = gi * len;
    const float* o = O + (size_t)r * ldo + c0;
    const float* z = P + (size_t)r * ldp + z_off + c0;
    // four channels per thread and load when everything is 16-byte aligned (the gated values stay in registers for rows up to 4096)
    const bool v4 = (len & 3) == 0 && (ldo & 3) == 0 && (ldp & 3) == 0 && ((z_off + c0) & 3) == 0 && (c0 & 3) == 0 && len <= 4 * 4 * 256;
    float4 keep[4];
    float ss = 0.0f;
    if (v4) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = (threadIdx.x + u * 256) * 4;
            keep[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < len) {
                const float4 a = *reinterpret_cast<const float4*>(o + c), g = *reinterpret_cast<const float4*>(z + c);
                keep[u] = make_float4(a.x * (g.x * sigmoid_f(g.x)), a.y * (g.y * sigmoid_f(g.y)), a.z * (g.z * sigmoid_f(g.z)), a.w * (g.w * sigmoid_f(g.w)));
                ss += keep[u].x * keep[u].x + keep[u].y * keep[u].y + keep[u].z * keep[u].z + keep[u].w * keep[u].w;
            }
        }
    } else {
        for (int c = threadIdx.x; c < len; c += blockDim.x) {
            const float v = o[c] * (z[c] * sigmoid_f(z[c]));
            ss = fmaf(v, v, ss);
        }
    }
    ss = wsum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
        red[8] = 1.0f / sqrtf(t / (float)len + eps);
    }
    __syncthreads();
    const float inv = red[8];
    if (v4) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = (threadIdx.x + u * 256) * 4;
            if (c < len) {
                const float4 wv = *reinterpret_cast<const float4*>(w + c0 + c);
                OutT* dst = out + (size_t)r * n + c0 + c;
                dst[0] = from_f<OutT>(keep[u].x * inv * wv.x);
                dst[1] = from_f<OutT>(keep[u].y * inv * wv.y);
                dst[2] = from_f<OutT>(keep[u].z * inv * wv.z);
                dst[3] = from_f<OutT>(keep[u].w * inv * wv.w);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < len; c += blockDim.x) {
        const float v = o[c] * (z[c] * sigmoid_f(z[c]));
        out[(size_t)r * n + c0 + c] = from_f<OutT>(v * inv * w[c0 + c]);
    }
}
