// The gated delta rule with one decay per key channel, and the per-head gated norm after it.
//
// Per head, with a state S [dim, vdim] in float32 that a sequence carries from token to token
// (zero when the sequence starts), a unit query q and key k [dim], a value v [vdim], a write
// strength beta and a decay g [dim] per token:
//     S <- diag(g) S;   e = beta * (v - S^T k);   S <- S + k e^T;   o = S^T q
// in this order, so that the read-out sees the token's own write.  Query and key arrive unnormalised
// (after their short convolution and silu) and are made unit vectors here, x / sqrt(sum x^2 + 1e-6),
// the query also times dim^-1/2.  The decay comes as the logit l of a low-rank projection:
// g = exp(-rate_h * softplus(l + dt)), rate_h = exp(A_h) made once.  beta = sigmoid of its logit.
// Value head h reads query/key head h / (heads / qk_heads).  Everything of the recurrence is 32-bit.
//
// delta_rule_prep makes unit q and k, decays and betas of all the step's tokens at once.
// delta_rule_scan: a sequence's new tokens are scanned in order from the state in its slot, which
// is updated in place: whole prompts, single tokens and anything between are one kernel.  Grid
// (heads * column groups of 8, sequences): sixteen neighbouring lanes share one column of S (a
// sixteenth of its rows in registers each) and add up the two sums over the column by shuffles, so that
// a single sequence still gives every SM several warps; q, k, g and v of a run of tokens are staged in
// shared memory, the next run's on their way meanwhile; the state's columns come and go through shared
// memory.
//
// head_gated_rmsnorm: y = o / rms(o) * w * act(gate) * out_scale per token and head over vdim, w [vdim] or none (ones);
//   act is the sigmoid or silu
// shared by the heads.
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int DR_TOK = 16;       // tokens staged at a time

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int DR_LPC = 16, DR_COLS = 8, DR_THREADS = DR_LPC * DR_COLS;      // sixteen lanes share a column of S; a block holds 8 columns

// What the recurrence needs of every token, made for all tokens at once: one warp per (token, unit); units 0 .. G - 1 are
// the query/key heads (unit vectors qn, kn [M, G, dim], the query times dim^-1/2), units G .. G + H - 1 the value heads
// (decays g [M, H, dim] and beta [M, H]).  All float32.
template <typename T>
__global__ void delta_rule_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, long long q_stride, long long k_stride,
                                       const float* __restrict__ decay_logit, const float* __restrict__ dt_bias,
                                       const float* __restrict__ rate, const T* __restrict__ beta_logit, long long beta_stride,
                                       float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ gg, float* __restrict__ beta,
                                       long long rows, int n_heads, int qk_heads, int dim) {
    ti_pdl_trigger();
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); decay_logit = ti_dependent(decay_logit); beta_logit = ti_dependent(beta_logit);
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= rows) return;
    const int lane = threadIdx.x & 31, units = qk_heads + n_heads;
    const long long m = w / units;
    const int unit = (int)(w - m * units);
    if (unit < qk_heads) {
        const T* qr = q + (size_t)m * q_stride + (size_t)unit * dim;
        const T* kr = k + (size_t)m * k_stride + (size_t)unit * dim;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < dim; i += 32) {
            const float a = to_f32(qr[i]), c = to_f32(kr[i]);
            sq = fmaf(a, a, sq);
            sk = fmaf(c, c, sk);
        }
        const float iq = rsqrtf(warp_sum(sq) + 1e-6f) * rsqrtf((float)dim), ik = rsqrtf(warp_sum(sk) + 1e-6f);
        float* qo = qn + ((size_t)m * qk_heads + unit) * dim;
        float* ko = kn + ((size_t)m * qk_heads + unit) * dim;
        for (int i = lane; i < dim; i += 32) { qo[i] = to_f32(qr[i]) * iq; ko[i] = to_f32(kr[i]) * ik; }
    } else {
        const int h = unit - qk_heads;
        const float rt = rate[h];
        const float* l = decay_logit + ((size_t)m * n_heads + h) * dim;
        float* go = gg + ((size_t)m * n_heads + h) * dim;
        for (int i = lane; i < dim; i += 32) go[i] = expf(-rt * softplus_f(l[i] + dt_bias[(size_t)h * dim + i]));
        if (lane == 0) beta[(size_t)m * n_heads + h] = 1.0f / (1.0f + expf(-to_f32(beta_logit[(size_t)m * beta_stride + h])));
    }
}

// Sixteen neighbouring lanes share a column of S: lane r holds the rows i = 16 NV jj + NV r + e (e < NV, jj < J; NV = 4
// and J = MAXD / 64 for heads of 64 and more), so that its q, k and g are reads of NV floats from shared memory, the
// sixteen lanes' reads side by side.  Staged rows are MAXD long, zero past dim, so that the inner loops have no bounds
// to check (rows of S past dim stay zero).  A run's operands are fetched into registers while the run before it is
// worked off.  (Measured on prompts of 2,048 tokens, 16 and 32 heads of 128 x 128: four lanes a column 1.64 and 1.88 ms,
// sixteen 1.00 and 1.03, a warp a column 0.77 and 1.52.)
template <int N> struct FloatRun { float x[N]; };

template <int N>
__device__ __forceinline__ FloatRun<N> lds_run(const float* p) {
    FloatRun<N> out;
    if constexpr (N == 4) { const float4 v = *reinterpret_cast<const float4*>(p); out.x[0] = v.x; out.x[1] = v.y; out.x[2] = v.z; out.x[3] = v.w; }
    else if constexpr (N == 2) { const float2 v = *reinterpret_cast<const float2*>(p); out.x[0] = v.x; out.x[1] = v.y; }
    else out.x[0] = *p;
    return out;
}

template <typename T, int MAXD>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ gg,
                       const float* __restrict__ beta, const T* __restrict__ v, long long v_stride,
                       float* __restrict__ o, float* __restrict__ state, long long slot_stride,
                       const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                       int n_heads, int qk_heads, int dim, int vdim, int groups) {
    ti_pdl_trigger();
    constexpr int NV = MAXD / DR_LPC >= 4 ? 4 : MAXD / DR_LPC, J = MAXD / (DR_LPC * NV), ROW = MAXD;
    constexpr int PIECES = 3 * DR_TOK * ROW / 4;                         // 16-byte pieces of a run's q, k, g
    constexpr int PER = (PIECES + DR_THREADS - 1) / DR_THREADS;
    extern __shared__ __align__(16) float sm[];                  // q, k, g: [DR_TOK][ROW] each; v: [DR_TOK][DR_COLS]; beta: [DR_TOK]
    ti_pdl_sync();
    qn = ti_dependent(qn); kn = ti_dependent(kn); gg = ti_dependent(gg); beta = ti_dependent(beta); v = ti_dependent(v);
    float* qs = sm;
    float* ks = qs + DR_TOK * ROW;
    float* gs = ks + DR_TOK * ROW;
    float* vs = gs + DR_TOK * ROW;
    float* bs = vs + DR_TOK * DR_COLS;
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0) return;
    const int hq = h / (n_heads / qk_heads);
    const int r = threadIdx.x & (DR_LPC - 1), cl = threadIdx.x / DR_LPC;
    const int col = g * DR_COLS + cl;
    const bool live = col < vdim;
    const bool vec = (dim & 3) == 0;
    float S[J][NV];
    float* srow = state + (size_t)seq_slot[b] * slot_stride + (size_t)h * dim * vdim;
    // the block's DR_COLS columns of S come and go through shared memory, so that global memory sees whole pieces of rows
    for (int idx = threadIdx.x; idx < dim * DR_COLS; idx += DR_THREADS) {
        const int i = idx / DR_COLS, c = g * DR_COLS + (idx - i * DR_COLS);
        sm[idx] = c < vdim ? srow[(size_t)i * vdim + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int jj = 0; jj < J; jj++)
#pragma unroll
        for (int e = 0; e < NV; e++) {
            const int i = DR_LPC * NV * jj + NV * r + e;
            S[jj][e] = i < dim ? sm[i * DR_COLS + cl] : 0.f;
        }
    float4 rr[PER];
    float rv = 0.f, rb = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(DR_TOK, n - t0);
#pragma unroll
        for (int p = 0; p < PER; p++) {
            const int idx = threadIdx.x + DR_THREADS * p;              // piece idx of [3][DR_TOK][ROW / 4]
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < PIECES) {
                const int which = idx / (DR_TOK * (ROW / 4)), rem = idx - which * (DR_TOK * (ROW / 4));
                const int tt = rem / (ROW / 4), i = 4 * (rem - tt * (ROW / 4));
                if (tt < nt && i < dim) {
                    const size_t tok = (size_t)(tok0 + t0 + tt);
                    const float* src = which == 0 ? qn + (tok * qk_heads + hq) * dim : which == 1 ? kn + (tok * qk_heads + hq) * dim
                                                                                                   : gg + (tok * n_heads + h) * dim;
                    if (vec) x = *reinterpret_cast<const float4*>(src + i);
                    else {
                        x.x = src[i];
                        if (i + 1 < dim) x.y = src[i + 1];
                        if (i + 2 < dim) x.z = src[i + 2];
                        if (i + 3 < dim) x.w = src[i + 3];
                    }
                }
            }
            rr[p] = x;
        }
        if (threadIdx.x < DR_TOK * DR_COLS) {
            const int tt = threadIdx.x / DR_COLS, c = g * DR_COLS + (threadIdx.x - tt * DR_COLS);
            rv = (tt < nt && c < vdim) ? to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + c]) : 0.f;
        }
        if (threadIdx.x < DR_TOK) rb = threadIdx.x < nt ? beta[(size_t)(tok0 + t0 + threadIdx.x) * n_heads + h] : 0.f;
    };
    fetch(0);
    for (int t0 = 0; t0 < n; t0 += DR_TOK) {
        const int nt = min(DR_TOK, n - t0);
        __syncthreads();             // the run before is worked off
#pragma unroll
        for (int p = 0; p < PER; p++)
            if (threadIdx.x + DR_THREADS * p < PIECES) reinterpret_cast<float4*>(sm)[threadIdx.x + DR_THREADS * p] = rr[p];
        if (threadIdx.x < DR_TOK * DR_COLS) vs[threadIdx.x] = rv;
        if (threadIdx.x < DR_TOK) bs[threadIdx.x] = rb;
        __syncthreads();
        if (t0 + DR_TOK < n) fetch(t0 + DR_TOK);          // on its way while this run is worked off
        // Token by token.  A warp issues in order, so the loop is arranged by hand: the next token's q, k, g are read
        // before this token's sums are waited for, and the sum for this token's output goes round the lanes together
        // with the next token's sum for its S^T k.
        auto rows_of = [&](const float* base, int tt, FloatRun<NV> (&x)[J]) {
#pragma unroll
            for (int jj = 0; jj < J; jj++) x[jj] = lds_run<NV>(base + tt * ROW + DR_LPC * NV * jj + NV * r);
        };
        auto decay_and_dot = [&](const FloatRun<NV> (&gv)[J], const FloatRun<NV> (&kv)[J]) {
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int jj = 0; jj < J; jj++)
#pragma unroll
                for (int e = 0; e < NV; e++) {
                    S[jj][e] *= gv[jj].x[e];
                    if (e & 1) d1 = fmaf(S[jj][e], kv[jj].x[e], d1); else d0 = fmaf(S[jj][e], kv[jj].x[e], d0);
                }
            return d0 + d1;
        };
        FloatRun<NV> kc[J], qc[J], gc[J];
        rows_of(ks, 0, kc); rows_of(qs, 0, qc); rows_of(gs, 0, gc);
        float dot = decay_and_dot(gc, kc);
        float bv = bs[0], vv = vs[cl];
#pragma unroll
        for (int sh = 1; sh < DR_LPC; sh <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sh);
        for (int tt = 0; tt < nt; tt++) {
            const bool more = tt + 1 < nt;
            const int nx = more ? tt + 1 : tt;
            FloatRun<NV> kx[J], qx[J], gx[J];
            rows_of(ks, nx, kx); rows_of(qs, nx, qx); rows_of(gs, nx, gx);
            const float bn = bs[nx], vn = vs[nx * DR_COLS + cl];
            const float e = bv * (vv - dot);
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int jj = 0; jj < J; jj++)
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    S[jj][i] = fmaf(kc[jj].x[i], e, S[jj][i]);
                    if (i & 1) a1 = fmaf(S[jj][i], qc[jj].x[i], a1); else a0 = fmaf(S[jj][i], qc[jj].x[i], a0);
                }
            float acc = a0 + a1;
            float nd = 0.f;
            if (more) nd = decay_and_dot(gx, kx);            // (the same for all lanes)
#pragma unroll
            for (int sh = 1; sh < DR_LPC; sh <<= 1) {
                acc += __shfl_xor_sync(0xffffffffu, acc, sh);
                nd += __shfl_xor_sync(0xffffffffu, nd, sh);
            }
            if (live && r == 0) o[(size_t)(tok0 + t0 + tt) * ((size_t)n_heads * vdim) + (size_t)h * vdim + col] = acc;
            dot = nd; bv = bn; vv = vn;
#pragma unroll
            for (int jj = 0; jj < J; jj++) { kc[jj] = kx[jj]; qc[jj] = qx[jj]; }
        }
    }
    __syncthreads();
#pragma unroll
    for (int jj = 0; jj < J; jj++)
#pragma unroll
        for (int e = 0; e < NV; e++) {
            const int i = DR_LPC * NV * jj + NV * r + e;
            if (i < dim) sm[i * DR_COLS + cl] = S[jj][e];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < dim * DR_COLS; idx += DR_THREADS) {
        const int i = idx / DR_COLS, c = g * DR_COLS + (idx - i * DR_COLS);
        if (c < vdim) srow[(size_t)i * vdim + c] = sm[idx];
    }
}

// one warp per (token, head)
template <typename T>
__global__ void head_gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                                          const float* __restrict__ w, T* __restrict__ out, long long out_stride, long long rows,
                                          int n_heads, int vdim, float eps, int gate_silu, float out_scale) {
    ti_pdl_trigger();
    ti_pdl_sync();
    o = ti_dependent(o); gate = ti_dependent(gate);
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long m = r / n_heads;
    const int h = (int)(r - m * n_heads);
    const float* orow = o + (size_t)r * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps) * out_scale;
    for (int i = lane; i < vdim; i += 32) {
        const float gl = to_f32(gate[(size_t)m * gate_stride + (size_t)h * vdim + i]);
        const float ga = (gate_silu ? gl : 1.0f) / (1.0f + expf(-gl));
        out[(size_t)m * out_stride + (size_t)h * vdim + i] = from_f32<T>(orow[i] * inv * (w ? w[i] : 1.0f) * ga);
    }
}

template <typename F>
int dispatch_dim(int dim, F&& f) {
    if (dim <= 32) return f(std::integral_constant<int, 32>());
    if (dim <= 64) return f(std::integral_constant<int, 64>());
    return f(std::integral_constant<int, 128>());
}

}  // namespace

// q, k: [M, qk_heads, dim] and v: [M, heads, vdim] of the engine's type (row strides given, heads dense); decay_logit:
// float32 [M, heads * dim]; dt_bias: float32 [heads * dim]; rate: float32 [heads]; beta_logit: [M, heads] (row stride
// given); o: float32 [M, heads * vdim]; state: float32, slot s at state + s * slot_stride holds [heads, dim, vdim];
// scratch: float32, M * (2 * qk_heads * dim + heads * dim + heads) values.
extern "C" int ti_delta_rule_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                  long long v_stride, const float* decay_logit, const float* dt_bias, const float* rate,
                                  const void* beta_logit, long long beta_stride, float* o, float* state, long long slot_stride,
                                  float* scratch, const int* cu_new, const int* seq_slot, int n_seq, int M, int n_heads,
                                  int qk_heads, int dim, int vdim, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || M == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && M > 0 && n_heads > 0 && qk_heads > 0 && n_heads % qk_heads == 0 && dim > 0 && vdim > 0 && scratch,
               "delta_rule_scan: bad sizes");
    TI_REQUIRE(dim <= 128, "delta_rule: heads of %d query/key elements are not supported (up to 128)", dim);
    const int groups = (vdim + DR_COLS - 1) / DR_COLS;
    float* qn = scratch;
    float* kn = qn + (size_t)M * qk_heads * dim;
    float* gg = kn + (size_t)M * qk_heads * dim;
    float* beta = gg + (size_t)M * n_heads * dim;
    const long long rows = (long long)M * (qk_heads + n_heads);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch(delta_rule_prep_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, (const T*)q, (const T*)k, q_stride,
                          k_stride, decay_logit, dt_bias, rate, (const T*)beta_logit, beta_stride, qn, kn, gg, beta, rows, n_heads, qk_heads, dim));
        TI_CHECK_LAUNCH("delta_rule_prep");
        return dispatch_dim(dim, [&](auto md) -> int {
            constexpr int MAXD = decltype(md)::value;
            constexpr size_t smem = (size_t)(3 * DR_TOK * MAXD + DR_TOK + DR_TOK * DR_COLS) * sizeof(float);
            TI_CUDA(ti_launch(delta_rule_scan_kernel<T, MAXD>, dim3(n_heads * groups, n_seq), dim3(DR_THREADS), smem, stream,
                              (const float*)qn, (const float*)kn, (const float*)gg, (const float*)beta, (const T*)v, v_stride, o, state,
                              slot_stride, cu_new, seq_slot, n_heads, qk_heads, dim, vdim, groups));
            TI_CHECK_LAUNCH("delta_rule_scan");
            return 0;
        });
    });
}

// o: float32 [M, heads * vdim]; gate: [M, heads * vdim] of the engine's type with row stride gate_stride; w: float32 [vdim]
// or null (ones); out: [M, heads * vdim] with row stride out_stride; gate_silu: the gate is silu(logit), else sigmoid(logit).
extern "C" int ti_head_gated_rmsnorm(const float* o, const void* gate, long long gate_stride, const float* w, void* out,
                                     long long out_stride, int M, int n_heads, int vdim, float eps, int gate_silu, float out_scale,
                                     int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && vdim > 0, "head_gated_rmsnorm: bad sizes");
    const long long rows = (long long)M * n_heads;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(head_gated_rmsnorm_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, o, (const T*)gate,
                                   gate_stride, w, (T*)out, out_stride, rows, n_heads, vdim, eps, gate_silu, out_scale));
        TI_CHECK_LAUNCH("head_gated_rmsnorm");
        return 0;
    });
}
