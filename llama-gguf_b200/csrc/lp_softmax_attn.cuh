// lp_softmax_attn.cuh — what the general softmax mixer (B200_MIX_SOFTMAX_ATTN) does between its fused input projection and the
// attention kernels of layerprog.cu: biases, the short causal convolution and its tail, rotary positions, the q / k norms, the
// blending of values across layers, and the write of the position's K / V rows into the slot's cache.  Included by layerprog.cu
// (inside its anonymous namespace, after StepMeta and AttnGeom).  Everything here is f32 in both compute modes; the rotation's
// angle, sine and cosine are evaluated in double (an f32 angle at a position in the thousands is off by 1e-4).
#pragma once

// Columns of the fused projection P: [q (H dim) | k (G dim) | v (G vdim) | gate ...]; the first C = (H + G) dim + G vdim of them
// pass through here.  State block of a run: tail [taps - 1][C] f32, the last projected rows (bias included) of the sequence.
struct PrepGeom {
    int C;                 // (H + G) dim + G vdim
    int taps;              // 0: no convolution (1: a weight per channel on the current input only)
    int qk_norm;           // B200_QKNORM_*
    int rot_dims;          // 0: no rotation
    int v_mix;             // B200_VMIX_*
    size_t rec_off;
    int rot_after_norm;    // 1: the q / k norm first, then the rotation
    float rot_gain;        // factor on cos and sin of the q / k rotation (stretched frequencies), 1 otherwise
    int v_rot;             // 1: the values are turned by their position (all pairs of a head, frequencies v_freq) before they are cached
};

// One block per row.  Step 1: u = P + bias, y = causal convolution of u over time (inputs before the run's first row come from the
// run's tail, zeros at the start of a sequence) into shared memory.  Step 2: per head of q and k (a warp each): rotate the first
// rot_dims channels (channel 2i with 2i + 1).  Step 3: the norm (over the whole of q and of k, or a warp per head).  Step 4: q to
// qbuf, k to the cache row, v (blended) to the cache row.  shift_tail: the step has one row per run and the block also moves the
// run's tail on by this row (else lp_attn_conv_tail_kernel does it for the whole run afterwards).  rot_after_norm swaps steps 2 and 3.
// v_rot: the pairs (2m, 2m + 1) of every value head are turned by pos * v_freq[m]; cos | sin of these angles also go to
// vrot_out[r][vdim], where the attention kernels find them to turn the summed values back.
__global__ void __launch_bounds__(256) lp_attn_prep2_kernel(StepMeta sm, AttnGeom a, PrepGeom g, const float* __restrict__ P, int ldp,
                                                            const float* __restrict__ bias, const float* __restrict__ cw,
                                                            const float* __restrict__ qw, const float* __restrict__ kw,
                                                            const double* __restrict__ inv_freq, const float* __restrict__ lam_p,
                                                            float* __restrict__ vsrc, float* __restrict__ qbuf, int shift_tail,
                                                            const double* __restrict__ v_freq, float* __restrict__ vrot_out) {
    extern __shared__ __align__(16) float ps[];
    float* y = ps;                              // [C]
    float* cs = ps + ((g.C + 3) & ~3);          // [rot_dims / 2] cos, then sin
    float* sn = cs + g.rot_dims / 2;
    float* vcs = cs + g.rot_dims;               // [vdim / 2] cos, then sin (v_rot)
    __shared__ float red[2][8];
    const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int run = sm.row_run[r], pos = sm.row_pos[r], t = r - sm.run_start[run];
    float* tail = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off);
    const int nt = g.taps;
    for (int c = threadIdx.x; c < g.C; c += blockDim.x) {
        const float b = bias ? bias[c] : 0.0f;
        float v;
        if (nt == 0) v = P[(size_t)r * ldp + c] + b;
        else {
            v = 0.0f;
            for (int i = 0; i < nt; i++) {
                const int tt = t - (nt - 1) + i;
                const float in = tt >= 0 ? P[(size_t)(r - t + tt) * ldp + c] + b : tail[(size_t)(nt - 1 + tt) * g.C + c];
                v = fmaf(cw[(size_t)c * nt + i], in, v);
            }
            if (shift_tail && nt > 1) {   // every run has one row (decoding): the tail moves on by this input, channel by channel
                for (int i = 0; i + 1 < nt - 1; i++) tail[(size_t)i * g.C + c] = tail[(size_t)(i + 1) * g.C + c];
                tail[(size_t)(nt - 2) * g.C + c] = P[(size_t)r * ldp + c] + b;
            }
        }
        y[c] = v;
    }
    for (int i = threadIdx.x; i < g.rot_dims / 2; i += blockDim.x) {
        double s, c;
        sincos((double)pos * inv_freq[i], &s, &c);
        cs[i] = (float)c * g.rot_gain;
        sn[i] = (float)s * g.rot_gain;
    }
    if (g.v_rot) {
        for (int i = threadIdx.x; i < a.vdim / 2; i += blockDim.x) {
            double s, c;
            sincos((double)pos * v_freq[i], &s, &c);
            vcs[i] = (float)c;
            vcs[a.vdim / 2 + i] = (float)s;
            vrot_out[(size_t)r * a.vdim + i] = (float)c;
            vrot_out[(size_t)r * a.vdim + a.vdim / 2 + i] = (float)s;
        }
    }
    __syncthreads();
    const int nq = a.H * a.dim, nk = a.G * a.dim;
    auto rotate_qk = [&]() {
        for (int h = warp; h < a.H + a.G; h += nw) {
            float* v = y + h * a.dim;
            for (int i = lane; i < g.rot_dims / 2; i += 32) {
                const float u0 = v[2 * i], u1 = v[2 * i + 1];
                v[2 * i] = u0 * cs[i] - u1 * sn[i];
                v[2 * i + 1] = u1 * cs[i] + u0 * sn[i];
            }
        }
        __syncthreads();
    };
    if (g.rot_dims > 0 && !g.rot_after_norm) rotate_qk();
    if (g.qk_norm == B200_QKNORM_WHOLE_WEIGHT) {   // one root mean square over all of q, one over all of k
        float sq = 0.0f, sk = 0.0f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) sq += y[c] * y[c];
        for (int c = threadIdx.x; c < nk; c += blockDim.x) sk += y[nq + c] * y[nq + c];
        sq = wsum(sq);
        sk = wsum(sk);
        if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
        __syncthreads();
        sq = 0.0f; sk = 0.0f;
        for (int i = 0; i < nw; i++) { sq += red[0][i]; sk += red[1][i]; }
        const float iq = 1.0f / sqrtf(sq / (float)nq + a.eps), ik = 1.0f / sqrtf(sk / (float)nk + a.eps);
        for (int c = threadIdx.x; c < nq; c += blockDim.x) y[c] = y[c] * iq * qw[c];
        for (int c = threadIdx.x; c < nk; c += blockDim.x) y[nq + c] = y[nq + c] * ik * kw[c];
    } else if (g.qk_norm == B200_QKNORM_HEAD_WEIGHT || g.qk_norm == B200_QKNORM_HEAD_UNIT) {
        for (int h = warp; h < a.H + a.G; h += nw) {
            float* v = y + h * a.dim;
            float ss = 0.0f;
            for (int d = lane; d < a.dim; d += 32) ss += v[d] * v[d];
            ss = wsum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)a.dim + a.eps);
            const float* w = g.qk_norm == B200_QKNORM_HEAD_WEIGHT ? (h < a.H ? qw : kw) : nullptr;
            for (int d = lane; d < a.dim; d += 32) v[d] = v[d] * inv * (w ? w[d] : 1.0f);
        }
    }
    __syncthreads();
    if (g.rot_dims > 0 && g.rot_after_norm) rotate_qk();
    if (g.v_rot) {
        const int half = a.vdim / 2;
        for (int i = threadIdx.x; i < a.G * half; i += blockDim.x) {
            const int hv = i / half, pm = i - hv * half;
            float* v = y + nq + nk + hv * a.vdim;
            const float u0 = v[2 * pm], u1 = v[2 * pm + 1];
            v[2 * pm] = u0 * vcs[pm] - u1 * vcs[half + pm];
            v[2 * pm + 1] = u1 * vcs[pm] + u0 * vcs[half + pm];
        }
        __syncthreads();
    }
    float* kc = reinterpret_cast<float*>(sm.run_kv[run] + a.kv_off) + (size_t)pos * nk;
    float* vc = reinterpret_cast<float*>(sm.run_kv[run] + a.kv_off) + (size_t)a.cap * nk + (size_t)pos * a.G * a.vdim;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) qbuf[(size_t)r * nq + c] = y[c];
    for (int c = threadIdx.x; c < nk; c += blockDim.x) kc[c] = y[nq + c];
    const int nv = a.G * a.vdim;
    const float lam = g.v_mix == B200_VMIX_BLEND ? *lam_p : 0.0f;
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        float v = y[nq + nk + c];
        if (g.v_mix == B200_VMIX_SOURCE) vsrc[(size_t)r * nv + c] = v;
        else if (g.v_mix == B200_VMIX_BLEND) v = (1.0f - lam) * v + lam * vsrc[(size_t)r * nv + c];
        vc[c] = v;
    }
}

// After the rows of a step have been convolved: the run's tail becomes the last taps - 1 inputs of (old tail ++ new rows + bias).
__global__ void lp_attn_conv_tail_kernel(StepMeta sm, PrepGeom g, const float* __restrict__ P, int ldp, const float* __restrict__ bias) {
    const int run = blockIdx.x, r0 = sm.run_start[run], len = sm.run_start[run + 1] - r0;
    float* tail = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off);
    for (int c = threadIdx.x; c < g.C; c += blockDim.x) {
        const float b = bias ? bias[c] : 0.0f;
        for (int i = 0; i < g.taps - 1; i++) {
            const int st = len + i - (g.taps - 1);
            tail[(size_t)i * g.C + c] = st >= 0 ? P[(size_t)(r0 + st) * ldp + c] + b : tail[(size_t)(i + len) * g.C + c];
        }
    }
}
