// lp_gated_recurrent.cuh — the recurrent branches of B200_MIX_ATTN_RECURRENT (a softmax mixer beside a recurrent unit on the same
// normed input), how the two branches meet, and the clamped gated feed-forward.  Included by layerprog.cu inside its anonymous
// namespace (after the scan helpers of the matrix memory).  Gates, states and norms are f32 in both compute modes.
#pragma once

// ------------------------------------------------------------------------------------------------ gated linear memory
// Per (run, head): S [dim][vdim] f32.  With q = silu(zq), f = l + (1 - l) sigmoid(zf + b) per key channel:
//   S <- diag(f) S + (1 - f) v^T,   o = S^T q          (the forget gate also says how much of v is written).
// lp_glin_gates_kernel turns the pre-activations zq, zf of all rows into q and f in place (once per row and channel: every block of
// the scan would otherwise repeat it for its few columns); the scan is laid out like the library's other scans: thread column j of
// S, the column cut into 16-channel pieces over neighbouring lanes, tokens staged a chunk at a time with 16-byte copies.
// State block of a run: S [H][dim][vdim].
// Long runs on an otherwise empty GPU are cut into `nseg` segments, because the update is affine in S with a diagonal factor:
//   MODE 1  every segment but the last folds its tokens from S = 0 into carry[run][seg + 1] (no outputs);
//   lp_glin_carry_kernel multiplies the forget gates of each segment per channel (D) and chains carry[k + 1] = D_k carry[k] +
//           carry[k + 1] from carry[0] = the state that earlier steps left, so that carry[k] is the state at the start of segment k;
//   MODE 2  every segment runs from its carry with outputs, the last one leaves the state.
// MODE 0 is the whole run in one block per column group (decoding, short runs, many runs).
struct GlinGeom {
    int H, dim, vdim;
    int q_off, v_off, f_off;   // columns of P
    size_t rec_off;
};
__global__ void lp_glin_gates_kernel(float* __restrict__ P, int ldp, GlinGeom g, const float* __restrict__ fb, const float* __restrict__ lower, int R) {
    const int n = g.H * g.dim;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * n) return;
    const int r = (int)(i / n), c = (int)(i - (size_t)r * n);
    float* p = P + (size_t)r * ldp;
    const float zq = p[g.q_off + c], lo = lower[c];
    p[g.q_off + c] = zq * sigmoid_f(zq);
    p[g.f_off + c] = lo + (1.0f - lo) * sigmoid_f(p[g.f_off + c] + fb[c]);
}
template <int DMAX, int MODE>
__global__ void __launch_bounds__(SCAN_BD) lp_gated_linear_kernel(StepMeta sm, GlinGeom g, const float* __restrict__ P, int ldp, int vec4,
                                                                  float* __restrict__ O, int ldo, int nseg, float* __restrict__ carry) {
    constexpr int CH = ScanChunk<DMAX>::N, SPLIT = DMAX / SCAN_DREG, COLS = SCAN_BD / SPLIT;
    __shared__ __align__(16) float qs[CH][DMAX];
    __shared__ __align__(16) float fs[CH][DMAX];
    __shared__ float vs[CH][COLS];
    const int tid = threadIdx.x, col = tid / SPLIT, sub = tid % SPLIT;
    const int j = blockIdx.x * COLS + col, h = blockIdx.y;
    const int zsegs = MODE == 1 ? nseg - 1 : MODE == 2 ? nseg : 1;
    const int run = blockIdx.z / zsegs, seg = blockIdx.z - run * zsegs;
    int r0 = sm.run_start[run], r1 = sm.run_start[run + 1];
    if (MODE != 0) {   // this block's segment of the run (it may be empty)
        const int sl = (r1 - r0 + nseg - 1) / nseg;
        r0 = min(r0 + seg * sl, r1);
        r1 = min(r0 + sl, r1);
    }
    const size_t hs = (size_t)g.dim * g.vdim;
    float* Sg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off) + (size_t)h * hs;
    float* Cin = MODE == 2 ? carry + (((size_t)run * nseg + seg) * g.H + h) * hs : nullptr;
    float* Sout = MODE == 0 ? Sg : MODE == 1 ? carry + (((size_t)run * nseg + seg + 1) * g.H + h) * hs : (seg == nseg - 1 ? Sg : nullptr);
    const float* Sin = MODE == 0 ? Sg : Cin;
    const bool live = j < g.vdim;
    float s[SCAN_DREG];
#pragma unroll
    for (int i = 0; i < SCAN_DREG; i++) {
        const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);   // channel of register i
        s[i] = (MODE != 1 && live && d < g.dim) ? Sin[(size_t)d * g.vdim + j] : 0.0f;
    }
    for (int i = tid; i < CH * DMAX; i += SCAN_BD) {   // beyond dim: q = 0 and f = 1, so the padding rows stay zero
        (&qs[0][0])[i] = 0.0f;
        (&fs[0][0])[i] = 1.0f;
    }
    const int jc = blockIdx.x * COLS + (tid % COLS);   // the column this thread stages
    const int d4 = g.dim >> 2;
    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();   // the previous chunk has been consumed
        if (vec4) {        // (dim, the columns' offsets and the row pitch are multiples of 4 floats)
            for (int i = tid; i < nt * d4; i += SCAN_BD) {
                const int t = i / d4, d = (i - t * d4) * 4;
                const float* p = P + (size_t)(c0 + t) * ldp + h * g.dim + d;
                if (MODE != 1) cp_async16(smem_u32(&qs[t][d]), p + g.q_off, 16u);
                cp_async16(smem_u32(&fs[t][d]), p + g.f_off, 16u);
            }
        } else {
            for (int t = 0; t < nt; t++) {
                const float* p = P + (size_t)(c0 + t) * ldp;
                for (int d = tid; d < g.dim; d += SCAN_BD) {
                    if (MODE != 1) cp_async4(&qs[t][d], p + g.q_off + h * g.dim + d);
                    cp_async4(&fs[t][d], p + g.f_off + h * g.dim + d);
                }
            }
        }
        for (int t = tid / COLS; t < nt; t += SPLIT) {
            if (jc < g.vdim) cp_async4(&vs[t][tid % COLS], P + (size_t)(c0 + t) * ldp + g.v_off + h * g.vdim + jc);
            else vs[t][tid % COLS] = 0.0f;
        }
        cp_async_wait_all();
        __syncthreads();
#pragma unroll 2
        for (int t = 0; t < nt; t++) {
            const float v = vs[t][col];
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_DREG; i += 4) {
                const float4 f4 = *reinterpret_cast<const float4*>(&fs[t][((i >> 2) * SPLIT + sub) * 4]);
                s[i] = fmaf(f4.x, s[i] - v, v);
                s[i + 1] = fmaf(f4.y, s[i + 1] - v, v);
                s[i + 2] = fmaf(f4.z, s[i + 2] - v, v);
                s[i + 3] = fmaf(f4.w, s[i + 3] - v, v);
                if (MODE != 1) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][((i >> 2) * SPLIT + sub) * 4]);
                    a0 = fmaf(s[i], q4.x, a0);
                    a1 = fmaf(s[i + 1], q4.y, a1);
                    a2 = fmaf(s[i + 2], q4.z, a2);
                    a3 = fmaf(s[i + 3], q4.w, a3);
                }
            }
            if (MODE != 1) {
                const float acc = split_sum<SPLIT>((a0 + a1) + (a2 + a3));
                if (live && sub == 0) O[(size_t)(c0 + t) * ldo + h * g.vdim + j] = acc;
            }
        }
    }
    if (live && Sout)
#pragma unroll
        for (int i = 0; i < SCAN_DREG; i++) {
            const int d = ((i >> 2) * SPLIT + sub) * 4 + (i & 3);
            if (d < g.dim) Sout[(size_t)d * g.vdim + j] = s[i];
        }
}

// The carries of a segmented run: block = (32 channels x 32 columns of a head's state, run).  First the product of the forget gates of every segment
// but the last, per channel (GC_TL threads walk a segment's tokens side by side; the gates are read in rows of 32 channels), then
// carry[0] = the state, carry[k + 1] = D_k carry[k] + carry[k + 1] over this block's part of the state.
constexpr int GC_CH = 32, GC_TL = 8, GC_SEG_MAX = 16;
__global__ void __launch_bounds__(GC_CH * GC_TL) lp_glin_carry_kernel(StepMeta sm, GlinGeom g, const float* __restrict__ P, int ldp, int nseg,
                                                                      float* __restrict__ carry) {
    __shared__ float part[GC_TL][GC_CH];
    __shared__ float D[GC_SEG_MAX][GC_CH];
    const int lane = threadIdx.x % GC_CH, tl = threadIdx.x / GC_CH;
    const int vt = (g.vdim + GC_CH - 1) / GC_CH;
    const int d0 = (blockIdx.x / vt) * GC_CH, v0 = (blockIdx.x % vt) * GC_CH, h = blockIdx.y, run = blockIdx.z;
    const int r0 = sm.run_start[run], r1 = sm.run_start[run + 1];
    const int sl = (r1 - r0 + nseg - 1) / nseg;
    const int d = d0 + lane;
    for (int k = 0; k + 1 < nseg; k++) {
        const int a = min(r0 + k * sl, r1), b = min(a + sl, r1);
        float prod = 1.0f;
        if (d < g.dim) {
#pragma unroll 4
            for (int t = a + tl; t < b; t += GC_TL) prod *= P[(size_t)t * ldp + g.f_off + h * g.dim + d];
        }
        part[tl][lane] = prod;
        __syncthreads();
        if (tl == 0) {
            float v = part[0][lane];
#pragma unroll
            for (int i = 1; i < GC_TL; i++) v *= part[i][lane];
            D[k][lane] = v;
        }
        __syncthreads();
    }
    const size_t hs = (size_t)g.dim * g.vdim;
    const float* Sg = reinterpret_cast<const float*>(sm.run_rec[run] + g.rec_off) + (size_t)h * hs;
    const int nd = min(GC_CH, g.dim - d0), nv = min(GC_CH, g.vdim - v0);
    for (int i = threadIdx.x; i < nd * nv; i += GC_CH * GC_TL) {
        const int dl = i / nv;
        const size_t at = (size_t)(d0 + dl) * g.vdim + v0 + (i - dl * nv);
        float* c = carry + ((size_t)run * nseg * g.H + h) * hs + at;
        const size_t step = (size_t)g.H * hs;
        float v = Sg[at];
        float fold[GC_SEG_MAX - 1];   // every segment's fold is fetched before the chain starts
#pragma unroll
        for (int k = 0; k < GC_SEG_MAX - 1; k++) fold[k] = k + 1 < nseg ? c[(size_t)(k + 1) * step] : 0.0f;
        c[0] = v;
#pragma unroll
        for (int k = 0; k < GC_SEG_MAX - 1; k++)
            if (k + 1 < nseg) {
                v = fmaf(D[k][dl], v, fold[k]);
                c[(size_t)(k + 1) * step] = v;
            }
    }
}

// ------------------------------------------------------------------------------------------------ gated unit
// One state per channel: z = sigmoid(zz + bz), u = zx + bx, c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), s <- (1 - z) s + z c;
// out = s * silu(zg) * out_scale in the compute type (the operand of the branch's output projection).  State block of a run: s [width].
// s_t = a_t s_(t-1) + b_t with a = 1 - z, b = z c is a composition of affine maps, so a run is cut into GU_SEG segments that
// blockDim.y threads per channel fold on their own (A = prod a, B = the segment's s from s = 0, both kept with the per-token (a, b)
// of short segments in registers); the carries are then chained in shared memory and every segment is walked once more from its
// true start.  One token per run (decoding) is one segment.
struct GunitGeom {
    int width;
    int z_off, x_off, g_off;   // columns of P
    size_t rec_off;
};
constexpr int GU_CH = 32, GU_SEG = 32;   // channels and segments per block
__device__ __forceinline__ void gunit_ab(float zz, float zx, float bz, float bx, float& a, float& b) {
    const float z = sigmoid_f(zz + bz), u = zx + bx;
    const float cand = u >= 0.0f ? u + 0.5f : sigmoid_f(u);
    a = 1.0f - z;
    b = z * cand;
}
template <typename OutT>
__global__ void __launch_bounds__(GU_CH * GU_SEG) lp_gated_unit_kernel(StepMeta sm, GunitGeom g, const float* __restrict__ P, int ldp,
                                                                        const float* __restrict__ zb, const float* __restrict__ xb,
                                                                        OutT* __restrict__ out, int out_ld, float out_scale) {
    __shared__ float As[GU_SEG][GU_CH], Bs[GU_SEG][GU_CH];
    const int c = blockIdx.x * GU_CH + threadIdx.x, seg = threadIdx.y, run = blockIdx.y;
    const int r0 = sm.run_start[run], len = sm.run_start[run + 1] - r0;
    float* sg = reinterpret_cast<float*>(sm.run_rec[run] + g.rec_off);
    const bool live = c < g.width;
    const int per = (len + GU_SEG - 1) / GU_SEG;
    const int t0 = min(seg * per, len), t1 = min(t0 + per, len);
    const float bz = live ? zb[c] : 0.0f, bx = live ? xb[c] : 0.0f;
    const float* pz = P + (size_t)r0 * ldp + g.z_off + c;
    const float* px = P + (size_t)r0 * ldp + g.x_off + c;
    float A = 1.0f, B = 0.0f;
    if (live && len > per) {   // (a single segment needs no first pass)
        int t = t0;
        for (; t + 4 <= t1; t += 4) {   // four tokens' loads in flight together
            float zz[4], zx[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                zz[u] = pz[(size_t)(t + u) * ldp];
                zx[u] = px[(size_t)(t + u) * ldp];
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float a, b;
                gunit_ab(zz[u], zx[u], bz, bx, a, b);
                A *= a;
                B = fmaf(a, B, b);
            }
        }
        for (; t < t1; t++) {
            float a, b;
            gunit_ab(pz[(size_t)t * ldp], px[(size_t)t * ldp], bz, bx, a, b);
            A *= a;
            B = fmaf(a, B, b);
        }
    }
    As[seg][threadIdx.x] = A;
    Bs[seg][threadIdx.x] = B;
    float s = live ? sg[c] : 0.0f;   // (read before the barrier: the last segment's thread overwrites it after its walk)
    __syncthreads();
    for (int q = 0; q < seg; q++) s = fmaf(As[q][threadIdx.x], s, Bs[q][threadIdx.x]);   // the state at the start of this segment
    if (!live) return;
    const float* pg = P + (size_t)r0 * ldp + g.g_off + c;
    OutT* po = out + (size_t)r0 * out_ld + c;
    int t = t0;
    for (; t + 4 <= t1; t += 4) {
        float zz[4], zx[4], zg[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            zz[u] = pz[(size_t)(t + u) * ldp];
            zx[u] = px[(size_t)(t + u) * ldp];
            zg[u] = pg[(size_t)(t + u) * ldp];
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float a, b;
            gunit_ab(zz[u], zx[u], bz, bx, a, b);
            s = fmaf(a, s, b);
            po[(size_t)(t + u) * out_ld] = from_f<OutT>(s * zg[u] * sigmoid_f(zg[u]) * out_scale);
        }
    }
    for (; t < t1; t++) {
        float a, b;
        gunit_ab(pz[(size_t)t * ldp], px[(size_t)t * ldp], bz, bx, a, b);
        s = fmaf(a, s, b);
        const float zg = pg[(size_t)t * ldp];
        po[(size_t)t * out_ld] = from_f<OutT>(s * zg * sigmoid_f(zg) * out_scale);
    }
    if (seg == (len - 1) / per) sg[c] = s;   // the last segment that holds tokens ends on the run's last state
}

// ------------------------------------------------------------------------------------------------ how the branches meet
// x[r] += weight * (a / rms(a) * wa + b / rms(b) * wb), a = ya[r], b = yb[r] the two branches' projected outputs; one block per row.
__global__ void __launch_bounds__(256) lp_dual_norm_add_kernel(float* __restrict__ x, const float* __restrict__ ya, const float* __restrict__ yb, int ldy,
                                                               const float* __restrict__ wa, const float* __restrict__ wb, int width, float eps,
                                                               float weight) {
    __shared__ float red[2][8];
    const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* a = ya + (size_t)r * ldy;
    const float* b = yb + (size_t)r * ldy;
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        sa = fmaf(a[c], a[c], sa);
        sb = fmaf(b[c], b[c], sb);
    }
    sa = wsum(sa);
    sb = wsum(sb);
    if (lane == 0) { red[0][warp] = sa; red[1][warp] = sb; }
    __syncthreads();
    sa = 0.0f; sb = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) { sa += red[0][i]; sb += red[1][i]; }
    const float ia = 1.0f / sqrtf(sa / (float)width + eps), ib = 1.0f / sqrtf(sb / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)r * width + c] += weight * (a[c] * ia * wa[c] + b[c] * ib * wb[c]);
}

// ------------------------------------------------------------------------------------------------ clamped gated feed-forward
// out[r][n] = g sigmoid(slope g) (u + 1), g = min(P[r][n], limit), u = clamp(P[r][ff + n], -limit, limit): P holds [gate | up].
// A thread takes VEC neighbouring units (VEC = 4: 16-byte loads; ff, the row pitch and the column offset multiples of 4).
__device__ __forceinline__ float clamped_glu_f(float zg, float zu, float limit, float slope) {
    const float g = fminf(zg, limit), u = fminf(fmaxf(zu, -limit), limit);
    return g * sigmoid_f(slope * g) * (u + 1.0f);
}
template <typename OutT, int VEC>
__global__ void lp_clamped_glu_kernel(const float* __restrict__ P, int ldp, OutT* __restrict__ out, int ff, int R, float limit, float slope) {
    const int per = ff / VEC;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * per) return;
    const int r = (int)(i / per), n = (int)(i - (size_t)r * per) * VEC;
    const float* p = P + (size_t)r * ldp;
    if (VEC == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p + n), b = *reinterpret_cast<const float4*>(p + ff + n);
        OutT* o = out + (size_t)r * ff + n;
        o[0] = from_f<OutT>(clamped_glu_f(a.x, b.x, limit, slope));
        o[1] = from_f<OutT>(clamped_glu_f(a.y, b.y, limit, slope));
        o[2] = from_f<OutT>(clamped_glu_f(a.z, b.z, limit, slope));
        o[3] = from_f<OutT>(clamped_glu_f(a.w, b.w, limit, slope));
    } else {
        out[(size_t)r * ff + n] = from_f<OutT>(clamped_glu_f(p[n], p[ff + n], limit, slope));
    }
}
