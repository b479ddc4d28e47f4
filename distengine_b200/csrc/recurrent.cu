// Mixers that carry a matrix state per head from token to token: the gated delta rule with a
// decay per key channel, and retention (a fixed decay per head, no softmax).  Both states live in
// float32 in the slot of their request; everything here is float32 arithmetic, the storage type T
// (float32 or bfloat16) is that of the projections that come in and of the rows that go out.
//
//   delta rule, per head, S [dk, dv]:   S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);
//                                       S <- S + k_t u^T;  o_t = S^T q_t
//   retention, per head:                S <- decay S + k_t v_t^T;  o_t = S^T q_t
//   generalized delta rule, per head:   S <- diag(w_t) S - z_t (k_t^T S) + k_t v_t^T;  o_t = S^T r_t
//                                       (both first terms read the old S; z_t = a_t k_t / (|k_t|^2
//                                       + 1e-6), which is (a_t u_t) u_t^T S for the unit key u_t)
//
// The columns of S never meet: column j needs k_t, q_t, g_t, beta_t and v_t[j] only.  The scan
// kernel therefore gives a column to four adjacent lanes (each holds a quarter of its rows in
// registers), so a token costs short chains of multiply-adds and butterfly sums over four lanes,
// and a block of up to 32 columns walks its sequence's tokens of the step one after the other
// while the next tokens' vectors arrive through cp.async.  The order of every sum depends on the
// head's sizes only: a state does not depend, bit for bit, on how its tokens were cut into steps.
//
// What is token-parallel runs before the scan in a kernel of its own: the short causal
// convolution over time with its activation (its last taps - 1 inputs are part of the slot's
// state), the unit norms of q and k, the gate beta and the decays for the delta rule; the rotation
// by position for retention.  After the scan one more kernel normalises every head's output by its
// root mean square and gates it.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------
// Before the delta rule: one block a token.
//   proj row = [q (G dk) | k (G dk) | v (H dv) | ...], b (H) from column b_col on: the stacked
//   projection's output
//   y[c] = silu(sum_j taps[c][j] * x[t - (K-1) + j][c]);  inputs before the step's first token of
//   the sequence come from the slot's state, conv_state[i] = input at position pos0 - (K-1) + i
//   (zeros at a sequence's start: the slot is zeroed at admission)
//   q, k: each head divided by sqrt(sum of squares + 1e-6); q times dk^-1/2
//   beta = sigmoid(b);  g = exp(-exp(A_log[h]) * softplus(a + dt_bias))
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void delta_prep_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ a,
                                  const float* __restrict__ taps, const float* __restrict__ dt_bias,
                                  const float* __restrict__ a_log, const float* __restrict__ state,
                                  long long slot_stride, int conv_offset,
                                  const int* __restrict__ token_seq,
                                  const int* __restrict__ token_slot,
                                  const int* __restrict__ positions,
                                  const int* __restrict__ seq_pos0, float* __restrict__ qn,
                                  float* __restrict__ kn, float* __restrict__ vv,
                                  float* __restrict__ beta, float* __restrict__ gdec, int H, int G,
                                  int dk, int dv, int K, int b_col) {
    extern __shared__ float sh[];                    // [2 G dk]
    const int n = blockIdx.x;
    const int qk = 2 * G * dk, C = qk + H * dv;
    const int seq = token_seq[n], slot = token_slot[n];
    const int off = positions[n] - seq_pos0[seq];   // the token's place in its sequence's portion
    pdl_wait();
    const float* cs = state + (size_t)slot * slot_stride + conv_offset;
#pragma unroll 2
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.0f;
#pragma unroll 4
        for (int j = 0; j < K; ++j) {
            const int rel = off - (K - 1) + j;
            const float x = rel >= 0 ? to_float(proj[(size_t)(n - (K - 1) + j) * ld + c])
                                     : cs[(size_t)(off + j) * C + c];
            acc = fmaf(taps[c * K + j], x, acc);
        }
        const float y = silu_f(acc);
        if (c < qk) sh[c] = y;
        else vv[(size_t)n * (H * dv) + (c - qk)] = y;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float q_scale = 1.0f / sqrtf((float)dk);
    for (int head = warp; head < 2 * G; head += warps) {
        const float* x = sh + head * dk;
        float ss = 0.0f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
        float* dst = head < G ? qn + (size_t)n * (G * dk) + head * dk
                              : kn + (size_t)n * (G * dk) + (head - G) * dk;
        for (int i = lane; i < dk; i += 32)
            dst[i] = head < G ? (x[i] * inv) * q_scale : x[i] * inv;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        beta[(size_t)n * H + h] = sigmoid_f(to_float(proj[(size_t)n * ld + b_col + h]));
    for (int i = threadIdx.x; i < H * dk; i += blockDim.x) {
        const float rate = expf(a_log[i / dk]);
        gdec[(size_t)n * (H * dk) + i] =
            expf(-rate * softplus_f(a[(size_t)n * (H * dk) + i] + dt_bias[i]));
    }
    pdl_trigger();
}

// After a step: the slot keeps the last K - 1 inputs of the convolution.  One block a sequence.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state,
                                  long long slot_stride, int conv_offset,
                                  const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_qstart,
                                  const int* __restrict__ seq_qlen, int C, int K) {
    const int s = blockIdx.x;
    const int qlen = seq_qlen[s], tok0 = seq_qstart[s];
    pdl_wait();
    pdl_trigger();
    float* cs = state + (size_t)seq_slot[s] * slot_stride + conv_offset;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        for (int i = 0; i < K - 1; ++i) {            // ascending: what is read lies ahead
            const int rel = qlen - (K - 1) + i;
            cs[(size_t)i * C + c] = rel >= 0 ? to_float(proj[(size_t)(tok0 + rel) * ld + c])
                                             : cs[(size_t)(i + qlen) * C + c];
        }
}

// ------------------------------------------------------------------------------------------
// Before retention: q and k rotated by position (pairs (i, i + rot/2) of the first `rot` features
// of a head, angle = float(position) * inv_freq[i], the rest unchanged), k times dk^-1/2 after.
//   proj row = [q (H dk) | k (H dk) | v | gate]; out: qr, kr float32 [N, H dk]
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void retention_prep_kernel(const T* __restrict__ proj, int ld,
                                      const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rot, int H, int dk,
                                      float* __restrict__ qr, float* __restrict__ kr) {
    const int n = blockIdx.x;
    const float pos = (float)positions[n];
    const int half = rot / 2, per = dk - half;      // work items a head: pairs, then plain features
    const float k_scale = 1.0f / sqrtf((float)dk);
    pdl_wait();
    for (int idx = threadIdx.x; idx < 2 * H * per; idx += blockDim.x) {
        const int which = idx / (H * per), rest = idx - which * (H * per);
        const int h = rest / per, i = rest - h * per;
        const T* src = proj + (size_t)n * ld + which * (H * dk) + h * dk;
        float* dst = (which ? kr : qr) + (size_t)n * (H * dk) + h * dk;
        const float scale = which ? k_scale : 1.0f;
        if (i < half) {
            float s, c;
            sincosf(pos * inv_freq[i], &s, &c);
            float ra, rb;
            rope_rotate(to_float(src[i]), to_float(src[i + half]), c, s, ra, rb);
            dst[i] = ra * scale;
            dst[i + half] = rb * scale;
        } else {
            dst[i + half] = to_float(src[i + half]) * scale;
        }
    }
    pdl_trigger();
}

// ------------------------------------------------------------------------------------------
// Before the generalized delta rule: one block a token.
//   proj row holds r, k, a (each H dk wide) from columns r_col, k_col, a_col on;
//   wl float32 [N, H dk]: the low-rank decay projection's output
//   rr = r, kk = k as float32;  w = exp(-exp(-1/2) * sigmoid(wl + w0))
//   z  = sigmoid(a + a_bias) * k / (sum over the head of k^2 + 1e-6)
//   dots [N, H, 2] = (z . r, k . r) per head: what the scan's read-out needs of them, the same for
//   every column of the state
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void gdelta_prep_kernel(const T* __restrict__ proj, int ld, int r_col, int k_col,
                                   int a_col, const float* __restrict__ wl,
                                   const float* __restrict__ w0, const float* __restrict__ a_bias,
                                   float* __restrict__ rr, float* __restrict__ kk,
                                   float* __restrict__ ww, float* __restrict__ zz,
                                   float* __restrict__ dots, int H, int dk) {
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* row = proj + (size_t)n * ld;
    const size_t base = (size_t)n * (H * dk);
    const float rate = 0.6065306597126334f;          // exp(-1/2)
    pdl_wait();
    for (int h = warp; h < H; h += warps) {
        const T* ks = row + k_col + h * dk;
        float ss = 0.0f;
        for (int i = lane; i < dk; i += 32) {
            const float x = to_float(ks[i]);
            ss = fmaf(x, x, ss);
        }
        const float inv2 = 1.0f / (warp_sum(ss) + 1e-6f);
        float zr = 0.0f, kr = 0.0f;
        for (int i = lane; i < dk; i += 32) {
            const int c = h * dk + i;
            const float x = to_float(ks[i]), r = to_float(row[r_col + c]);
            const float z = sigmoid_f(to_float(row[a_col + c]) + a_bias[c]) * x * inv2;
            kk[base + c] = x;
            rr[base + c] = r;
            zz[base + c] = z;
            ww[base + c] = expf(-rate * sigmoid_f(wl[base + c] + w0[c]));
            zr = fmaf(z, r, zr);
            kr = fmaf(x, r, kr);
        }
        zr = warp_sum(zr);
        kr = warp_sum(kr);
        if (lane == 0) {
            dots[((size_t)n * H + h) * 2] = zr;
            dots[((size_t)n * H + h) * 2 + 1] = kr;
        }
    }
    pdl_trigger();
}

// silu of `cols` columns of proj into float32 [N, cols] (queries and keys of a mixer without any
// other preparation).
template <typename T>
__global__ void silu_rows_kernel(const T* __restrict__ proj, int ld, float* __restrict__ out,
                                 int cols, size_t total) {
    pdl_wait();
    pdl_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / cols;
        const int i = (int)(idx - n * cols);
        out[idx] = silu_f(to_float(proj[n * ld + i]));
    }
}

// ------------------------------------------------------------------------------------------
// The scan.  grid (sequences, heads, column blocks of COLS); a column belongs to LANES = 4
// adjacent lanes; thread = LANES * column + share.
// Rows of the state go to the shares four at a time: row i belongs to share (i / 4) % LANES,
// register 4 * (i / (4 LANES)) + i % 4; in shared memory a token's vector lies share by share
// (share l at l * (R + 4)), so four consecutive rows are 16 bytes there as in memory (one
// cp.async), a share reads its rows as float4 and the shares of a warp hit different banks.  COLS is 32, or less when a step has so few (sequence, head) pairs that blocks of 32
// columns would leave most SMs idle.  A sequence's blocks also move the slot's kept convolution
// inputs on, a share of the channels each (`conv_*`; the kernel before this one has read the old
// ones).
// ------------------------------------------------------------------------------------------
constexpr int TB = 8;          // tokens whose vectors are in flight together

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

struct ConvKeep {              // the convolution inputs a slot keeps (K <= 1: nothing to do)
    const void* proj;
    int ld, bf16, offset, C, K;
};

template <int LANES>
__device__ __forceinline__ int state_row(int r, int l) {      // register r of share l -> row
    return (r >> 2) * (4 * LANES) + (l << 2) + (r & 3);
}

// MODE 0: retention; 1: the delta rule (g, beta); 2: the generalized delta rule (g = w, z).
template <typename VT, int R, int MODE, int COLS, int LANES>
// (the generalized rule at 32 columns is held to three blocks an SM: single tokens stream the
// states, and 183 registers a thread would leave two)
__global__ void __launch_bounds__(COLS * LANES, (MODE == 2 && R <= 32 && COLS == 32) ? 3 : 1)
scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
            const VT* __restrict__ v, int ldv, const float* __restrict__ g, int ldg,
            const float* __restrict__ beta, int ldb, const float* __restrict__ z, int ldz,
            const float* __restrict__ decay,
            float* __restrict__ state, long long slot_stride, float* __restrict__ out,
            const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
            const int* __restrict__ seq_qlen, int H, int rep, int dk, int dv, int vec16,
            ConvKeep keep) {
    constexpr int PD = LANES * (R + 4);                  // a token's vector in shared memory
    constexpr bool DELTA = MODE == 1;
    constexpr int VECS = MODE == 0 ? 2 : (MODE == 1 ? 3 : 4);      // q, k (, g (, z))
    extern __shared__ __align__(16) float buf[];     // [2][TB][VECS][PD]
    const int s = blockIdx.x, h = blockIdx.y;
    const int col = blockIdx.z * COLS + threadIdx.x / LANES, l = threadIdx.x % LANES;
    const bool live = col < dv;
    const int qlen = seq_qlen[s], tok0 = seq_qstart[s];
    const int hk = h / rep;                          // the q/k head this head reads
    if (dk < LANES * R) {                            // rows beyond dk: their q, k, g stay zero
        for (int i = threadIdx.x; i < 2 * TB * VECS * PD; i += COLS * LANES) buf[i] = 0.0f;
        __syncthreads();
    }
    pdl_wait();
    // (The state through shared memory, so that memory sees whole rows of COLS columns, was
    // measured and is slower: 92 against 55 us for 64 single tokens of 16 heads of 128 x 128.)

    float* slot_state = state + (size_t)seq_slot[s] * slot_stride;
    if (keep.K > 1) {                                // the sequence's blocks share the channels out
        float* cs = slot_state + keep.offset;
        const int rank = h * gridDim.z + blockIdx.z, blocks = H * gridDim.z;
        for (int c = rank * (COLS * LANES) + threadIdx.x; c < keep.C; c += blocks * (COLS * LANES))
            for (int i = 0; i < keep.K - 1; ++i) {   // ascending: what is read lies ahead
                const int rel = qlen - (keep.K - 1) + i;
                float x;
                if (rel < 0) x = cs[(size_t)(i + qlen) * keep.C + c];
                else if (keep.bf16)
                    x = __bfloat162float(((const __nv_bfloat16*)keep.proj)[(size_t)(tok0 + rel) * keep.ld + c]);
                else x = ((const float*)keep.proj)[(size_t)(tok0 + rel) * keep.ld + c];
                cs[(size_t)i * keep.C + c] = x;
            }
    }
    float* S_g = slot_state + (size_t)h * dk * dv;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = state_row<LANES>(r, l);
        S[r] = (live && i < dk) ? S_g[(size_t)i * dv + col] : 0.0f;
    }
    const float dec = MODE == 0 ? decay[h] : 0.0f;

    auto issue = [&](int b) {
        float* dst = buf + (size_t)(b & 1) * TB * VECS * PD;
        const int count = min(TB, qlen - b * TB);
        if (vec16) {
            const int quads = dk >> 2;
            for (int idx = threadIdx.x; idx < count * quads; idx += COLS * LANES) {
                const int t = idx / quads, c = idx - t * quads;
                const size_t tok = (size_t)(tok0 + b * TB + t);
                float* d = dst + (size_t)t * VECS * PD + (c % LANES) * (R + 4) + ((c / LANES) << 2);
                cp_async16(d, q + tok * ldq + hk * dk + 4 * c);
                cp_async16(d + PD, k + tok * ldk + hk * dk + 4 * c);
                if (MODE >= 1) cp_async16(d + 2 * PD, g + tok * ldg + h * dk + 4 * c);
                if (MODE == 2) cp_async16(d + 3 * PD, z + tok * ldz + h * dk + 4 * c);
            }
        } else {
            for (int idx = threadIdx.x; idx < count * dk; idx += COLS * LANES) {
                const int t = idx / dk, i = idx - t * dk;
                const size_t tok = (size_t)(tok0 + b * TB + t);
                float* d = dst + (size_t)t * VECS * PD + ((i >> 2) % LANES) * (R + 4) +
                           (((i >> 2) / LANES) << 2) + (i & 3);
                cp_async4(d, q + tok * ldq + hk * dk + i);
                cp_async4(d + PD, k + tok * ldk + hk * dk + i);
                if (MODE >= 1) cp_async4(d + 2 * PD, g + tok * ldg + h * dk + i);
                if (MODE == 2) cp_async4(d + 3 * PD, z + tok * ldz + h * dk + i);
            }
        }
        cp_async_commit();
    };
    // a batch's values and gates do not depend on the state: they are asked for a batch ahead
    float nv[TB], nb[TB], nc[TB];
    auto fetch = [&](int b) {
        const int count = min(TB, qlen - b * TB);
#pragma unroll
        for (int t = 0; t < TB; ++t) {
            const size_t tok = (size_t)(tok0 + b * TB + t);
            nv[t] = (live && t < count) ? to_float(v[tok * ldv + h * dv + col]) : 0.0f;
            nb[t] = (DELTA && t < count) ? beta[tok * ldb + h] : 0.0f;
            if (MODE == 2) {                         // (z . r, k . r) of the token's head
                nb[t] = t < count ? beta[tok * ldb + 2 * h] : 0.0f;
                nc[t] = t < count ? beta[tok * ldb + 2 * h + 1] : 0.0f;
            }
        }
    };

    const int batches = (qlen + TB - 1) / TB;
    if (batches > 0) {
        issue(0);
        fetch(0);
    }
    for (int b = 0; b < batches; ++b) {
        const int count = min(TB, qlen - b * TB);
        float vt[TB], bt[TB], ct[TB];
#pragma unroll
        for (int t = 0; t < TB; ++t) {
            vt[t] = nv[t];
            bt[t] = nb[t];
            ct[t] = MODE == 2 ? nc[t] : 0.0f;
        }
        if (b + 1 < batches) {
            issue(b + 1);
            fetch(b + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* src = buf + (size_t)(b & 1) * TB * VECS * PD + l * (R + 4);
#pragma unroll
        for (int t = 0; t < TB; ++t) {
            if (t >= count) break;
            const float4* q4 = reinterpret_cast<const float4*>(src + (size_t)t * VECS * PD);
            const float4* k4 = reinterpret_cast<const float4*>(src + (size_t)t * VECS * PD + PD);
            // The read-out needs no second pass over the new state: with D = diag(g) S,
            //   S' = D + k u^T  and  o = S'^T q = D^T q + u (k . q),
            // so D^T k, D^T q and k . q are summed together (three sums over the quarter's rows,
            // one butterfly over the four quarters for all three) and the update of S is the
            // last thing a token does, off the next token's critical path but for S itself.
            if (MODE == 2) {
                // With p = k^T S (old state) the new state is diag(w) S - z p + k v and the
                // read-out (w S)^T r - p (z . r) + v (k . r); z . r and k . r do not depend on the
                // column and come with the token.  Two sums in one pass over the quarter's rows,
                // one butterfly for both, the update of S last.
                const float4* w4 =
                    reinterpret_cast<const float4*>(src + (size_t)t * VECS * PD + 2 * PD);
                const float4* z4 =
                    reinterpret_cast<const float4*>(src + (size_t)t * VECS * PD + 3 * PD);
                float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const float4 ww = w4[r], kk = k4[r], qq = q4[r];
                    p0 = fmaf(S[4 * r + 0], kk.x, p0); S[4 * r + 0] *= ww.x; a0 = fmaf(S[4 * r + 0], qq.x, a0);
                    p1 = fmaf(S[4 * r + 1], kk.y, p1); S[4 * r + 1] *= ww.y; a1 = fmaf(S[4 * r + 1], qq.y, a1);
                    p2 = fmaf(S[4 * r + 2], kk.z, p2); S[4 * r + 2] *= ww.z; a2 = fmaf(S[4 * r + 2], qq.z, a2);
                    p3 = fmaf(S[4 * r + 3], kk.w, p3); S[4 * r + 3] *= ww.w; a3 = fmaf(S[4 * r + 3], qq.w, a3);
                }
                float p = (p0 + p1) + (p2 + p3), o = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int step = 1; step < LANES; step <<= 1) {
                    p += __shfl_xor_sync(0xffffffffu, p, step);
                    o += __shfl_xor_sync(0xffffffffu, o, step);
                }
                const float val = vt[t];
                o = fmaf(val, ct[t], fmaf(-p, bt[t], o));
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const float4 kk = k4[r], zz = z4[r];
                    S[4 * r + 0] = fmaf(-zz.x, p, fmaf(kk.x, val, S[4 * r + 0]));
                    S[4 * r + 1] = fmaf(-zz.y, p, fmaf(kk.y, val, S[4 * r + 1]));
                    S[4 * r + 2] = fmaf(-zz.z, p, fmaf(kk.z, val, S[4 * r + 2]));
                    S[4 * r + 3] = fmaf(-zz.w, p, fmaf(kk.w, val, S[4 * r + 3]));
                }
                if (live && l == 0)
                    out[(size_t)(tok0 + b * TB + t) * (H * dv) + h * dv + col] = o;
                continue;
            }
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
            float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;      // k . q
            float u;
            if (DELTA) {
                const float4* g4 =
                    reinterpret_cast<const float4*>(src + (size_t)t * VECS * PD + 2 * PD);
                float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const float4 gg = g4[r], kk = k4[r], qq = q4[r];
                    S[4 * r + 0] *= gg.x; p0 = fmaf(S[4 * r + 0], kk.x, p0); o0 = fmaf(S[4 * r + 0], qq.x, o0); c0 = fmaf(kk.x, qq.x, c0);
                    S[4 * r + 1] *= gg.y; p1 = fmaf(S[4 * r + 1], kk.y, p1); o1 = fmaf(S[4 * r + 1], qq.y, o1); c1 = fmaf(kk.y, qq.y, c1);
                    S[4 * r + 2] *= gg.z; p2 = fmaf(S[4 * r + 2], kk.z, p2); o2 = fmaf(S[4 * r + 2], qq.z, o2); c2 = fmaf(kk.z, qq.z, c2);
                    S[4 * r + 3] *= gg.w; p3 = fmaf(S[4 * r + 3], kk.w, p3); o3 = fmaf(S[4 * r + 3], qq.w, o3); c3 = fmaf(kk.w, qq.w, c3);
                }
                float part = (p0 + p1) + (p2 + p3);
                part += __shfl_xor_sync(0xffffffffu, part, 1);
                part += __shfl_xor_sync(0xffffffffu, part, 2);
                if (LANES == 8) part += __shfl_xor_sync(0xffffffffu, part, 4);
                u = bt[t] * (vt[t] - part);
            } else {
                u = vt[t];
#pragma unroll
                for (int r = 0; r < R / 4; ++r) {
                    const float4 kk = k4[r], qq = q4[r];
                    S[4 * r + 0] *= dec; o0 = fmaf(S[4 * r + 0], qq.x, o0); c0 = fmaf(kk.x, qq.x, c0);
                    S[4 * r + 1] *= dec; o1 = fmaf(S[4 * r + 1], qq.y, o1); c1 = fmaf(kk.y, qq.y, c1);
                    S[4 * r + 2] *= dec; o2 = fmaf(S[4 * r + 2], qq.z, o2); c2 = fmaf(kk.z, qq.z, c2);
                    S[4 * r + 3] *= dec; o3 = fmaf(S[4 * r + 3], qq.w, o3); c3 = fmaf(kk.w, qq.w, c3);
                }
            }
            float o = (o0 + o1) + (o2 + o3), kq = (c0 + c1) + (c2 + c3);
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            kq += __shfl_xor_sync(0xffffffffu, kq, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            kq += __shfl_xor_sync(0xffffffffu, kq, 2);
            if (LANES == 8) {
                o += __shfl_xor_sync(0xffffffffu, o, 4);
                kq += __shfl_xor_sync(0xffffffffu, kq, 4);
            }
            o = fmaf(u, kq, o);
#pragma unroll
            for (int r = 0; r < R / 4; ++r) {
                const float4 kk = k4[r];
                S[4 * r + 0] = fmaf(kk.x, u, S[4 * r + 0]);
                S[4 * r + 1] = fmaf(kk.y, u, S[4 * r + 1]);
                S[4 * r + 2] = fmaf(kk.z, u, S[4 * r + 2]);
                S[4 * r + 3] = fmaf(kk.w, u, S[4 * r + 3]);
            }
            if (live && l == 0)
                out[(size_t)(tok0 + b * TB + t) * (H * dv) + h * dv + col] = o;
        }
        __syncthreads();                             // the buffer may be filled again
    }
    pdl_trigger();
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = state_row<LANES>(r, l);
            if (i < dk) S_g[(size_t)i * dv + col] = S[r];
        }
    }
}

// ------------------------------------------------------------------------------------------
// After the scan: every head's output over its root mean square, gated.  A warp a (token, head).
//   mode 0: out = o / rms * weight[j] * sigmoid(gate)   gate float32 [N, H dv]
//   mode 1: out = o / rms * silu(gate)                  gate of type T, row stride ld_gate
//   mode 2: out = o / rms * weight[h dv + j] * sigmoid(gate)   gate of type T; the weight spans
//           all heads (with H = 1 the root mean square is that of the whole row)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ o, const void* __restrict__ gate,
                                 int ld_gate, const float* __restrict__ weight,
                                 T* __restrict__ out, int n_tokens, int H, int dv, float eps,
                                 int mode) {
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_wait();
    pdl_trigger();
    if (item >= n_tokens * H) return;
    const int n = item / H, h = item - n * H;
    const float* x = o + (size_t)n * (H * dv) + h * dv;
    float ss = 0.0f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    T* dst = out + (size_t)n * (H * dv) + h * dv;
    for (int j = lane; j < dv; j += 32) {
        float y = x[j] * inv;
        if (mode == 0) {
            const float gt = ((const float*)gate)[(size_t)n * ld_gate + h * dv + j];
            y = y * weight[j] * sigmoid_f(gt);
        } else if (mode == 1) {
            const float gt = to_float(((const T*)gate)[(size_t)n * ld_gate + h * dv + j]);
            y = y * silu_f(gt);
        } else {
            const float gt = to_float(((const T*)gate)[(size_t)n * ld_gate + h * dv + j]);
            y = y * weight[h * dv + j] * sigmoid_f(gt);
        }
        dst[j] = from_float<T>(y);
    }
}

// out = (a / rms(a) * wa + b / rms(b) * wb) / 2 over the model width.  One block a token.
template <typename T>
__global__ void mean_of_normed_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                      const float* __restrict__ wa, const float* __restrict__ wb,
                                      T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    pdl_wait();
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(a[base + i]), y = to_float(b[base + i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, scratch) / (float)width + eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, scratch) / (float)width + eps);
    pdl_trigger();
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(a[base + i]) * ia * wa[i];
        const float y = to_float(b[base + i]) * ib * wb[i];
        out[base + i] = from_float<T>(0.5f * (x + y));
    }
}

// The same with a single head as wide as the row (one root mean square a token, the weight over
// the row, sigmoid of a gate of type T): one block a token.
template <typename T>
__global__ void row_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ld_gate,
                                const float* __restrict__ weight, T* __restrict__ out, int dv,
                                float eps) {
    __shared__ float scratch[33];
    const int n = blockIdx.x;
    const float* x = o + (size_t)n * dv;
    pdl_wait();
    float ss = 0.0f;
    for (int j = threadIdx.x; j < dv; j += blockDim.x) ss = fmaf(x[j], x[j], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dv + eps);
    pdl_trigger();
    for (int j = threadIdx.x; j < dv; j += blockDim.x)
        out[(size_t)n * dv + j] = from_float<T>(
            x[j] * inv * weight[j] * sigmoid_f(to_float(gate[(size_t)n * ld_gate + j])));
}

template <typename VT, int MODE, int COLS, int LANES>
int launch_scan_cols(int R, dim3 grid, cudaStream_t s, const float* q, int ldq, const float* k,
                     int ldk, const VT* v, int ldv, const float* g, int ldg, const float* beta,
                     int ldb, const float* z, int ldz, const float* decay, float* state, long long slot_stride, float* out,
                     const int* seq_slot, const int* seq_qstart, const int* seq_qlen, int H,
                     int rep, int dk, int dv, int vec16, ConvKeep keep) {
#define SCAN(RR)                                                                                \
    do {                                                                                        \
        const size_t smem = (size_t)2 * TB * (MODE + 2) * LANES * (RR + 4) * sizeof(float);     \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(scan_kernel<VT, RR, MODE, COLS, LANES>,        \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        return de_launch(scan_kernel<VT, RR, MODE, COLS, LANES>, grid, dim3(COLS * LANES),      \
                         smem, s, q, ldq, k, ldk, v, ldv, g, ldg, beta, ldb, z, ldz, decay, state, \
                         slot_stride, out, seq_slot, seq_qstart, seq_qlen, H, rep, dk, dv,      \
                         vec16, keep);                                                          \
    } while (0)
    if (R <= 8) SCAN(8);
    if (R <= 16) SCAN(16);
    if (R <= 32) SCAN(32);
    if (LANES == 4) SCAN(64);
    return -6;
#undef SCAN
}

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            count = 148;
    }
    return count;
}

template <typename VT, int MODE>
int launch_scan(cudaStream_t s, const float* q, int ldq, const float* k, int ldk, const VT* v,
                int ldv, const float* g, int ldg, const float* beta, int ldb, const float* z,
                int ldz, const float* decay,
                float* state, long long slot_stride, float* out, const int* seq_slot,
                const int* seq_qstart, const int* seq_qlen, int n_seqs, int H, int rep, int dk,
                int dv, ConvKeep keep) {
    const int vec16 = (dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && (MODE == 0 || ldg % 4 == 0) &&
                       (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                       (MODE == 0 || (uintptr_t)g % 16 == 0) &&
                       (MODE != 2 || (ldz % 4 == 0 && (uintptr_t)z % 16 == 0))) ? 1 : 0;
    const long long pairs = (long long)n_seqs * H;
#define COLS_CASE(CC, LL)                                                                       \
    return launch_scan_cols<VT, MODE, CC, LL>(R, grid, s, q, ldq, k, ldk, v, ldv, g, ldg,       \
                                               beta, ldb, z, ldz, decay, state, slot_stride, out, \
                                               seq_slot, seq_qstart, seq_qlen, H, rep, dk, dv, \
                                               vec16, keep)
    // (eight lanes a column - twice the warps, half the instructions a token and warp - was
    // measured for a single long prompt and is slower: 867 against 788 us for 2,048 tokens of 16
    // heads of 128 x 128; a token's time is its chain of dependent steps, which a third butterfly
    // stage lengthens)
    const int R = 4 * ((dk + 15) / 16);
    // narrower blocks while blocks of 32 columns would not give every SM two
    int cols = 32;
    while (cols > 8 && pairs * ((dv + cols - 1) / cols) < 2LL * sm_count()) cols >>= 1;
    dim3 grid(n_seqs, H, (dv + cols - 1) / cols);
    if (cols == 8) COLS_CASE(8, 4);
    if (cols == 16) COLS_CASE(16, 4);
    COLS_CASE(32, 4);
#undef COLS_CASE
}

}  // namespace

DE_EXPORT int de_recurrent_max_key_dim() { return 256; }

DE_EXPORT int de_delta_prep(int dtype, const void* proj, int ld, const float* a, const float* taps,
                            const float* dt_bias, const float* a_log, const float* state,
                            long long slot_stride, int conv_offset, const int* token_seq,
                            const int* token_slot, const int* positions, const int* seq_pos0,
                            float* qn, float* kn, float* vv, float* beta, float* gdec, int n, int H,
                            int G, int dk, int dv, int K, int b_col, void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || K <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)2 * G * dk * sizeof(float);
    if (smem > 200 * 1024) return -3;
    if (smem > 48 * 1024) {
        const cudaError_t e =
            dtype == DE_BF16
                ? cudaFuncSetAttribute(delta_prep_kernel<__nv_bfloat16>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                : cudaFuncSetAttribute(delta_prep_kernel<float>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // a block a token: many threads, so that a token of a decode step is a few rounds of loads
    // (with few tokens: steps of many tokens fill the GPU with blocks of 256)
    const int work = 2 * G * dk + H * dv;
    const int threads = n >= 512 ? 256 : (work >= 4096 ? 1024 : (work >= 1024 ? 512 : 256));
#define PREP(T)                                                                                 \
    return de_launch(delta_prep_kernel<T>, dim3(n), dim3(threads), smem, s, (const T*)proj, ld, a,  \
                     taps, dt_bias, a_log, state, slot_stride, conv_offset, token_seq,          \
                     token_slot, positions, seq_pos0, qn, kn, vv, beta, gdec, H, G, dk, dv, K,  \
                     b_col)
    if (dtype == DE_BF16) PREP(__nv_bfloat16);
    PREP(float);
#undef PREP
}

DE_EXPORT int de_conv_state(int dtype, const void* proj, int ld, float* state,
                            long long slot_stride, int conv_offset, const int* seq_slot,
                            const int* seq_qstart, const int* seq_qlen, int n_seqs, int C, int K,
                            void* stream) {
    if (n_seqs <= 0 || K <= 1) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16)
        return de_launch(conv_state_kernel<__nv_bfloat16>, dim3(n_seqs), dim3(256), 0, s,
                         (const __nv_bfloat16*)proj, ld, state, slot_stride, conv_offset, seq_slot,
                         seq_qstart, seq_qlen, C, K);
    return de_launch(conv_state_kernel<float>, dim3(n_seqs), dim3(256), 0, s, (const float*)proj,
                     ld, state, slot_stride, conv_offset, seq_slot, seq_qstart, seq_qlen, C, K);
}

DE_EXPORT int de_retention_prep(int dtype, const void* proj, int ld, const int* positions,
                                const float* inv_freq, int rot, int H, int dk, float* qr, float* kr,
                                int n, void* stream) {
    if (n <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > dk) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = n >= 512 ? 256 : (2 * H * dk >= 2048 ? 1024 : (2 * H * dk >= 512 ? 512 : 256));
    if (dtype == DE_BF16)
        return de_launch(retention_prep_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s,
                         (const __nv_bfloat16*)proj, ld, positions, inv_freq, rot, H, dk, qr, kr);
    return de_launch(retention_prep_kernel<float>, dim3(n), dim3(threads), 0, s,
                     (const float*)proj, ld, positions, inv_freq, rot, H, dk, qr, kr);
}

// v_dtype: the type of v (DE_F32 for the delta rule, whose values come from its own preparation).
// mode 1: g [N, ldg] and beta [N, ldb] are used (the delta rule); 2: g (the decays w), z
// [N, ldz] and in beta's place the heads' (z . r, k . r) [N, 2 H] (the generalized delta rule);
// 0: decay [H].  conv_taps > 1: the slots also keep the
// last conv_taps - 1 rows of the first conv_channels columns of conv_proj (of type conv_dtype,
// row stride conv_ld) at conv_offset of their state row.
DE_EXPORT int de_state_scan(int mode, int v_dtype, const float* q, int ldq, const float* k,
                            int ldk, const void* v, int ldv, const float* g, int ldg,
                            const float* beta, int ldb, const float* z, int ldz,
                            const float* decay, float* state, long long slot_stride, float* out,
                            const int* seq_slot, const int* seq_qstart, const int* seq_qlen,
                            int n_seqs, int H, int rep, int dk, int dv, const void* conv_proj,
                            int conv_ld, int conv_dtype, int conv_offset, int conv_channels,
                            int conv_taps, void* stream) {
    if (n_seqs <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || H <= 0 || rep <= 0 || H % rep) return -2;
    if (mode < 0 || mode > 2) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    ConvKeep keep = {conv_proj, conv_ld, conv_dtype == DE_BF16 ? 1 : 0, conv_offset,
                     conv_channels, conv_proj ? conv_taps : 0};
#define SCAN_ARGS(VT)                                                                           \
    s, q, ldq, k, ldk, (const VT*)v, ldv, g, ldg, beta, ldb, z, ldz, decay, state, slot_stride, \
        out, seq_slot, seq_qstart, seq_qlen, n_seqs, H, rep, dk, dv, keep
    if (mode == 1) {
        if (v_dtype != DE_F32) return -4;
        return launch_scan<float, 1>(SCAN_ARGS(float));
    }
    if (mode == 2) {
        if (rep != 1) return -2;
        if (v_dtype == DE_BF16) return launch_scan<__nv_bfloat16, 2>(SCAN_ARGS(__nv_bfloat16));
        return launch_scan<float, 2>(SCAN_ARGS(float));
    }
    if (v_dtype == DE_BF16) return launch_scan<__nv_bfloat16, 0>(SCAN_ARGS(__nv_bfloat16));
    return launch_scan<float, 0>(SCAN_ARGS(float));
#undef SCAN_ARGS
}

DE_EXPORT int de_gdelta_prep(int dtype, const void* proj, int ld, int r_col, int k_col, int a_col,
                             const float* wl, const float* w0, const float* a_bias, float* rr,
                             float* kk, float* ww, float* zz, float* dots, int n, int H, int dk,
                             void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || dk <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = n >= 512 ? 128 : (H >= 8 ? 256 : 32 * (H < 1 ? 1 : H));
    if (dtype == DE_BF16)
        return de_launch(gdelta_prep_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s,
                         (const __nv_bfloat16*)proj, ld, r_col, k_col, a_col, wl, w0, a_bias, rr,
                         kk, ww, zz, dots, H, dk);
    return de_launch(gdelta_prep_kernel<float>, dim3(n), dim3(threads), 0, s, (const float*)proj,
                     ld, r_col, k_col, a_col, wl, w0, a_bias, rr, kk, ww, zz, dots, H, dk);
}

DE_EXPORT int de_silu_rows(int dtype, const void* proj, int ld, float* out, int n, int cols,
                           void* stream) {
    if (n <= 0 || cols <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)n * cols;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == DE_BF16)
        return de_launch(silu_rows_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s,
                         (const __nv_bfloat16*)proj, ld, out, cols, total);
    return de_launch(silu_rows_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s,
                     (const float*)proj, ld, out, cols, total);
}

DE_EXPORT int de_head_gate(int dtype, const float* o, const void* gate, int ld_gate,
                           const float* weight, void* out, int n, int H, int dv, float eps,
                           int mode, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == 2 && H == 1 && dv > 256) {
        const int threads = dv >= 2048 ? 512 : 256;
        if (dtype == DE_BF16)
            return de_launch(row_gate_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s, o,
                             (const __nv_bfloat16*)gate, ld_gate, weight, (__nv_bfloat16*)out, dv,
                             eps);
        return de_launch(row_gate_kernel<float>, dim3(n), dim3(threads), 0, s, o,
                         (const float*)gate, ld_gate, weight, (float*)out, dv, eps);
    }
    const int warps = 4;
    dim3 grid((n * H + warps - 1) / warps);
    if (dtype == DE_BF16)
        return de_launch(head_gate_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, s, o, gate,
                         ld_gate, weight, (__nv_bfloat16*)out, n, H, dv, eps, mode);
    return de_launch(head_gate_kernel<float>, grid, dim3(warps * 32), 0, s, o, gate, ld_gate,
                     weight, (float*)out, n, H, dv, eps, mode);
}

DE_EXPORT int de_mean_of_normed(int dtype, const void* a, const void* b, const float* wa,
                                const float* wb, void* out, int n, int width, float eps,
                                void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == DE_BF16)
        return de_launch(mean_of_normed_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s,
                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, wa, wb,
                         (__nv_bfloat16*)out, width, eps);
    return de_launch(mean_of_normed_kernel<float>, dim3(n), dim3(threads), 0, s, (const float*)a,
                     (const float*)b, wa, wb, (float*)out, width, eps);
}
