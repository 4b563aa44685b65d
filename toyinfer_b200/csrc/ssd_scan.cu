// The selective state-space recurrence of Mamba-2 (state-space duality: Dao and Gu, "Transformers
// are SSMs") and the gated norm after it.  32-bit throughout: step sizes, decays, the state and
// everything that enters it are float32 whatever the engine's type.
//
// Per head h (group g = h / (heads / groups)), with x_t [vdim], B_t and C_t [N] of the group (all
// three out of the short convolution and its silu), dt_t the head's raw step size:
//     d_t = softplus(dt_t + dt_bias[h]);   a_t = exp(-rate[h] * d_t)        (rate = exp(A_log))
//     S_t = a_t S_(t-1) + d_t B_t x_t^T     (S is N x vdim, zero when the sequence starts)
//     y_t = S_t^T C_t + D[h] x_t
// The state of a sequence lives in its slot as [heads, vdim, N] (a column's N values side by
// side).  ssd_scan walks a sequence's new tokens in order from the state the slot holds and
// leaves it as it is after them, however many tokens the step brings (a prompt, a piece, one).
// Grid (column groups of 32, heads, sequences), 128 threads: a column's N values are shared out
// over 8 lanes (R consecutive values a lane, two columns a thread, so that a read of B and C
// serves both), whose partial sums of y meet by three shuffles for both columns; B, C, x
// and the step sizes of a run of 16 tokens are staged in shared memory, the next run's fetched
// into registers meanwhile (16 bytes a read where the rows allow it).
// Long prompts are cut into segments that run in parallel (the recurrence is linear in the state
// and a segment's decays multiply to one number per head): a first launch finds every segment's own
// effect on a zero state, a second walks each sequence's segments and leaves every segment's start
// state, the third runs the recurrence of all segments at once.
//
// gate_group_rmsnorm: v = y * silu(z);  v / rms(v) over each of `groups` equal parts of the row,
// times a weight per channel.
#include "common.cuh"

#include <algorithm>
#include <type_traits>

namespace {

constexpr int SCAN_THREADS = 128, LPC = 8, CPT = 2, COLS = SCAN_THREADS / LPC * CPT, RUN = 16;      // CPT: columns a thread

__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// R consecutive floats of shared memory, 16 bytes a read (8 for R = 2)
template <int R>
__device__ __forceinline__ void row_values(const float* __restrict__ p, float (&x)[R]) {
    if constexpr (R >= 4) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
            const float4 q = *reinterpret_cast<const float4*>(p + r);
            x[r] = q.x; x[r + 1] = q.y; x[r + 2] = q.z; x[r + 3] = q.w;
        }
    } else {
        const float2 q = *reinterpret_cast<const float2*>(p);
        x[0] = q.x; x[1] = q.y;
    }
}

// OUT: the recurrence with its outputs, from the state the slot holds (n_seg == 1) or from the segment's start state in
// `scratch`; the last segment of a sequence leaves the state in the slot.  !OUT: a segment's own effect on a state that
// starts at zero, for every segment but a sequence's last: the end state goes to scratch[b * n_seg + p + 1], the product
// of its decays to seg_decay[(b * n_seg + p) * heads + h].  `vec`: rows can be read 16 bytes at a time; the next run's
// rows are then fetched into registers while this run is worked off.
template <typename T, int R, bool OUT>
__global__ void __launch_bounds__(SCAN_THREADS)
ssd_scan_kernel(const T* __restrict__ xbc, long long ld_xbc, const T* __restrict__ dt_raw, long long ld_dt,
                const float* __restrict__ dt_bias, const float* __restrict__ rate, const float* __restrict__ skip,
                float* __restrict__ state, long long slot_stride, float* __restrict__ y, const int* __restrict__ cu_new,
                const int* __restrict__ seq_slot, int heads, int groups, int N, int vdim, int seg, int n_seg,
                float* __restrict__ scratch, float* __restrict__ seg_decay, int vec) {
    ti_pdl_trigger();
    constexpr int NP = LPC * R;                  // N rounded up to what the lanes hold
    constexpr int CH = R >= 4 ? 4 : 2;           // floats of one read or write of shared memory
    constexpr int RP = R + CH;                   // a lane's R values lie side by side, lanes RP apart: no bank is hit twice
    constexpr int PITCH = LPC * RP;              // floats of a token's row of B (or C) in shared memory
    constexpr int VEC = 16 / (int)sizeof(T);     // elements of a 16-byte read
    constexpr int NV = (RUN * NP / VEC + SCAN_THREADS - 1) / SCAN_THREADS;      // such reads per thread, run and operand
    constexpr int NX = RUN * COLS / SCAN_THREADS;
    extern __shared__ __align__(16) float sm[];
    float* Bs = sm;                              // [RUN][PITCH]: value n of a token at (n / R) * RP + n % R
    float* Cs = Bs + RUN * PITCH;                // [RUN][PITCH]
    float* xs = Cs + RUN * PITCH;                // [RUN][COLS]
    float* ds = xs + RUN * COLS;                 // [RUN] step sizes
    float* as = ds + RUN;                        // [RUN] decays
    const int b = blockIdx.z / n_seg, p = blockIdx.z - b * n_seg;
    const int h = blockIdx.y, v0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, col = tid / LPC, sub = tid % LPC;
    const int v = v0 + col * CPT;                // this thread's first column
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const float hb = dt_bias[h], hr = rate[h], hd = skip ? skip[h] : 0.f;
    for (int i = tid; i < 2 * RUN * PITCH; i += SCAN_THREADS) sm[i] = 0.f;   // values from N on stay zero
    ti_pdl_sync();
    xbc = ti_dependent(xbc); dt_raw = ti_dependent(dt_raw);
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    const int t_begin = p * seg, t_end = min(n, t_begin + seg);
    if (n <= 0 || t_begin >= t_end) return;
    const bool last = t_end == n;
    if (!OUT && last) return;
    const size_t per_slot = (size_t)inner * N, at = ((size_t)h * vdim + v) * N;
    float* slot_st = state + (size_t)seq_slot[b] * slot_stride + at;
    float S[CPT][R];
#pragma unroll
    for (int c = 0; c < CPT; c++)
#pragma unroll
        for (int r = 0; r < R; r++) S[c][r] = 0.f;
    // a lane's R values of a column are read and written 16 bytes at a time where the column holds all of them and starts
    // on such a boundary (a step of single tokens is this read and this write and little else)
    const bool whole = R >= 4 && N % 4 == 0 && slot_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0 &&
                       (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 15) == 0) && sub * R + R <= N;
    if (OUT) {
        const float* from = scratch ? scratch + (size_t)(b * n_seg + p) * per_slot + at : slot_st;
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            if constexpr (R >= 4) {
                if (whole && v + c < vdim) {
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        const float4 q = __ldcs(reinterpret_cast<const float4*>(from + (size_t)c * N + sub * R + r));
                        S[c][r] = q.x; S[c][r + 1] = q.y; S[c][r + 2] = q.z; S[c][r + 3] = q.w;
                    }
                    continue;
                }
            }
#pragma unroll
            for (int r = 0; r < R; r++) S[c][r] = (v + c < vdim && sub * R + r < N) ? from[(size_t)c * N + sub * R + r] : 0.f;
        }
    }
    const T* Bg = xbc + inner + (size_t)g * N;
    const T* Cg = xbc + inner + (size_t)(groups + g) * N;
    const int nvr = max(1, N / VEC);             // 16-byte reads per row (vec)
    uint4 pb[NV], pc[NV];
    T px[NX], pdt;
    auto fetch = [&](int t0) {
        const int nt = min(RUN, t_end - t0);
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int idx = tid + k * SCAN_THREADS, t = idx / nvr, jv = idx - t * nvr;
            pb[k] = make_uint4(0, 0, 0, 0); pc[k] = make_uint4(0, 0, 0, 0);
            if (t < nt) {
                const size_t row = (size_t)(tok0 + t0 + t) * ld_xbc + (size_t)jv * VEC;
                pb[k] = *reinterpret_cast<const uint4*>(Bg + row);
                if (OUT) pc[k] = *reinterpret_cast<const uint4*>(Cg + row);
            }
        }
#pragma unroll
        for (int k = 0; k < NX; k++) {
            const int idx = tid + k * SCAN_THREADS, t = idx / COLS, c = idx - t * COLS;
            px[k] = (t < nt && v0 + c < vdim) ? xbc[(size_t)(tok0 + t0 + t) * ld_xbc + (size_t)h * vdim + v0 + c] : from_f32<T>(0.f);
        }
        pdt = tid < nt ? dt_raw[(size_t)(tok0 + t0 + tid) * ld_dt + h] : from_f32<T>(0.f);
    };
    auto put = [&](float* dst, const T* e) {     // CH values side by side
        if constexpr (CH == 4) *reinterpret_cast<float4*>(dst) = make_float4(to_f32(e[0]), to_f32(e[1]), to_f32(e[2]), to_f32(e[3]));
        else *reinterpret_cast<float2*>(dst) = make_float2(to_f32(e[0]), to_f32(e[1]));
    };
    double log_decay = 0.0;
    if (vec) fetch(t_begin);
    for (int t0 = t_begin; t0 < t_end; t0 += RUN) {
        const int nt = min(RUN, t_end - t0);
        __syncthreads();        // the run before is used up
        if (vec) {
#pragma unroll
            for (int k = 0; k < NV; k++) {
                const int idx = tid + k * SCAN_THREADS, t = idx / nvr, jv = idx - t * nvr;
                if (t < RUN) {
                    const T* eb = reinterpret_cast<const T*>(&pb[k]);
                    const T* ec = reinterpret_cast<const T*>(&pc[k]);
#pragma unroll
                    for (int e = 0; e < VEC; e += CH) {      // (N is a multiple of VEC here, and R of CH: a chunk stays with one lane)
                        const int j = jv * VEC + e, at_j = t * PITCH + (j / R) * RP + j % R;
                        put(Bs + at_j, eb + e);
                        if (OUT) put(Cs + at_j, ec + e);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < NX; k++) xs[tid + k * SCAN_THREADS] = to_f32(px[k]);
            if (tid < RUN) {
                const float d = softplusf(to_f32(pdt) + hb);
                ds[tid] = d;
                as[tid] = expf(-hr * d);
            }
        } else {
            for (int idx = tid; idx < nt * N; idx += SCAN_THREADS) {
                const int t = idx / N, j = idx - t * N, at_j = t * PITCH + (j / R) * RP + j % R;
                const size_t row = (size_t)(tok0 + t0 + t) * ld_xbc;
                Bs[at_j] = to_f32(Bg[row + j]);
                if (OUT) Cs[at_j] = to_f32(Cg[row + j]);
            }
            for (int idx = tid; idx < nt * COLS; idx += SCAN_THREADS) {
                const int t = idx / COLS, c = idx - t * COLS;
                xs[idx] = v0 + c < vdim ? to_f32(xbc[(size_t)(tok0 + t0 + t) * ld_xbc + (size_t)h * vdim + v0 + c]) : 0.f;
            }
            if (tid < nt) {
                const float d = softplusf(to_f32(dt_raw[(size_t)(tok0 + t0 + tid) * ld_dt + h]) + hb);
                ds[tid] = d;
                as[tid] = expf(-hr * d);
            }
        }
        __syncthreads();
        if (vec && t0 + RUN < t_end) fetch(t0 + RUN);
        for (int t = 0; t < nt; t++) {
            const float a = as[t], d = ds[t];
            const float2 xv = *reinterpret_cast<const float2*>(xs + t * COLS + col * CPT);
            const float dx0 = d * xv.x, dx1 = d * xv.y;
            float Bt[R];
            row_values<R>(Bs + t * PITCH + sub * RP, Bt);
            if (OUT) {
                float Ct[R];
                row_values<R>(Cs + t * PITCH + sub * RP, Ct);
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    S[0][r] = fmaf(a, S[0][r], dx0 * Bt[r]);
                    S[1][r] = fmaf(a, S[1][r], dx1 * Bt[r]);
                    acc0 = fmaf(S[0][r], Ct[r], acc0);
                    acc1 = fmaf(S[1][r], Ct[r], acc1);
                }
                // the eight lanes' sums of both columns in three exchanges: even lanes go on with the first column,
                // odd lanes with the second
                const bool odd = sub & 1;
                float mine = (odd ? acc1 : acc0) + __shfl_xor_sync(0xffffffffu, odd ? acc0 : acc1, 1);
                mine += __shfl_xor_sync(0xffffffffu, mine, 2);
                mine += __shfl_xor_sync(0xffffffffu, mine, 4);
                if (sub < CPT && v + sub < vdim)
                    y[(size_t)(tok0 + t0 + t) * inner + (size_t)h * vdim + v + sub] = fmaf(hd, odd ? xv.y : xv.x, mine);
            } else {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    S[0][r] = fmaf(a, S[0][r], dx0 * Bt[r]);
                    S[1][r] = fmaf(a, S[1][r], dx1 * Bt[r]);
                }
            }
        }
        if (!OUT && tid == 0)
            for (int t = 0; t < nt; t++) log_decay -= (double)hr * (double)ds[t];
    }
    float* to = OUT ? (last ? slot_st : nullptr) : scratch + (size_t)(b * n_seg + p + 1) * per_slot + at;
    if (to != nullptr) {
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            if constexpr (R >= 4) {
                if (whole && v + c < vdim) {
#pragma unroll
                    for (int r = 0; r < R; r += 4)
                        *reinterpret_cast<float4*>(to + (size_t)c * N + sub * R + r) = make_float4(S[c][r], S[c][r + 1], S[c][r + 2], S[c][r + 3]);
                    continue;
                }
            }
#pragma unroll
            for (int r = 0; r < R; r++)
                if (v + c < vdim && sub * R + r < N) to[(size_t)c * N + sub * R + r] = S[c][r];
        }
    }
    if (!OUT && blockIdx.x == 0 && tid == 0) seg_decay[(size_t)(b * n_seg + p) * heads + h] = (float)exp(log_decay);
}

// The start state of every segment of a sequence, from the slot's state and the segments' own effects and decays:
// scratch[b, 0] = the slot's; scratch[b, p + 1] = decay[b, p] * scratch[b, p] + (what ssd_scan_kernel<.., false> left there).
__global__ void ssd_segment_carry_kernel(const float* __restrict__ state, long long slot_stride, float* __restrict__ scratch,
                                         const float* __restrict__ seg_decay, const int* __restrict__ cu_new,
                                         const int* __restrict__ seq_slot, int heads, int per_head, int seg, int n_seg) {
    ti_pdl_trigger();
    ti_pdl_sync();
    scratch = ti_dependent(scratch); seg_decay = ti_dependent(seg_decay);
    const int b = blockIdx.y;
    const int n = cu_new[b + 1] - cu_new[b];
    if (n <= 0) return;
    const int segs = (n + seg - 1) / seg;
    const size_t per_slot = (size_t)heads * per_head;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_slot; i += (size_t)gridDim.x * blockDim.x) {
        const int h = (int)(i / per_head);
        float s = state[(size_t)seq_slot[b] * slot_stride + i];
        float* sc = scratch + (size_t)b * n_seg * per_slot + i;
        sc[0] = s;
        for (int p = 0; p + 1 < segs; p++) {
            s = fmaf(seg_decay[(size_t)(b * n_seg + p) * heads + h], s, sc[(size_t)(p + 1) * per_slot]);
            sc[(size_t)(p + 1) * per_slot] = s;
        }
    }
}

template <typename T>
__global__ void gate_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ldz,
                                          const float* __restrict__ w, T* __restrict__ out, int inner, int groups, float eps) {
    ti_pdl_trigger();
    __shared__ float red[33];
    ti_pdl_sync();
    y = ti_dependent(y); z = ti_dependent(z);
    const int m = blockIdx.x, gs = inner / groups, base = blockIdx.y * gs;
    const float* yr = y + (size_t)m * inner + base;
    const T* zr = z + (size_t)m * ldz + base;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float zi = to_f32(zr[i]);
        const float u = yr[i] * (zi / (1.0f + expf(-zi)));
        ss = fmaf(u, u, ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float zi = to_f32(zr[i]);
        const float u = yr[i] * (zi / (1.0f + expf(-zi)));
        out[(size_t)m * inner + base + i] = from_f32<T>(u * inv * w[base + i]);
    }
}

}  // namespace

// xbc: [M, heads * vdim + 2 * groups * N] of the engine's type (x, then B, then C), row stride ld_xbc; dt_raw: [M, heads],
// row stride ld_dt; dt_bias, rate, skip: float32 [heads] (skip may be null); state: float32, slot s at
// state + s * slot_stride holds [heads, vdim, N]; y: float32 dense [M, heads * vdim].
// n_seg > 1: every sequence's new tokens are cut into segments of `seg` tokens (n_seg >= the longest sequence's count)
// that run in parallel: each segment's own effect on a zero state, a walk over a sequence's segments that gives each
// its start state, then the recurrence itself per segment.  scratch: float32 [n_seq * n_seg, heads * vdim * N];
// seg_decay: float32 [n_seq * n_seg, heads].  Three launches instead of one.
extern "C" int ti_ssd_scan(const void* xbc, long long ld_xbc, const void* dt_raw, long long ld_dt, const float* dt_bias,
                           const float* rate, const float* skip, float* state, long long slot_stride, float* y, const int* cu_new,
                           const int* seq_slot, int n_seq, int heads, int groups, int N, int vdim, int seg, int n_seg,
                           float* scratch, float* seg_decay, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && heads > 0 && heads <= 65535 && groups > 0 && heads % groups == 0 && N > 0 && vdim > 0, "ssd_scan: bad sizes");
    TI_REQUIRE(N <= LPC * 32, "ssd_scan: a state of %d values per column is not supported (up to %d)", N, LPC * 32);
    TI_REQUIRE(n_seg >= 1 && (long long)n_seq * n_seg <= 65535 && (n_seg == 1 || (seg > 0 && scratch && seg_decay)),
               "ssd_scan: %d sequences in %d segments", n_seq, n_seg);
    if (n_seg == 1) { seg = 1 << 30; scratch = nullptr; }
    const int rows = (N + LPC - 1) / LPC;
    const int inner = heads * vdim;
    dim3 grid((vdim + COLS - 1) / COLS, heads, n_seq * n_seg);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        constexpr int VEC = 16 / (int)sizeof(T);
        const int vec = (N % VEC == 0 && inner % VEC == 0 && ld_xbc % VEC == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0) ? 1 : 0;
        auto go = [&](auto rv) -> int {
            constexpr int R = decltype(rv)::value;
            const size_t smem = ((size_t)2 * RUN * LPC * (R + (R >= 4 ? 4 : 2)) + RUN * COLS + 2 * RUN) * sizeof(float);
            if (n_seg > 1) {
                TI_CUDA(ti_launch(ssd_scan_kernel<T, R, false>, grid, dim3(SCAN_THREADS), smem, stream, (const T*)xbc, ld_xbc, (const T*)dt_raw,
                                  ld_dt, dt_bias, rate, skip, state, slot_stride, y, cu_new, seq_slot, heads, groups, N, vdim, seg, n_seg,
                                  scratch, seg_decay, vec));
                TI_CHECK_LAUNCH("ssd_scan (segments)");
                const long long per_slot = (long long)inner * N;
                TI_CUDA(ti_launch(ssd_segment_carry_kernel, dim3((unsigned)std::min<long long>((per_slot + 255) / 256, 1024), n_seq), dim3(256), 0,
                                  stream, (const float*)state, slot_stride, scratch, (const float*)seg_decay, cu_new, seq_slot, heads,
                                  vdim * N, seg, n_seg));
                TI_CHECK_LAUNCH("ssd_scan (carry)");
            }
            TI_CUDA(ti_launch(ssd_scan_kernel<T, R, true>, grid, dim3(SCAN_THREADS), smem, stream, (const T*)xbc, ld_xbc, (const T*)dt_raw, ld_dt,
                              dt_bias, rate, skip, state, slot_stride, y, cu_new, seq_slot, heads, groups, N, vdim, seg, n_seg, scratch,
                              seg_decay, vec));
            TI_CHECK_LAUNCH("ssd_scan");
            return 0;
        };
        if (rows <= 2) return go(std::integral_constant<int, 2>());
        if (rows <= 4) return go(std::integral_constant<int, 4>());
        if (rows <= 8) return go(std::integral_constant<int, 8>());
        if (rows <= 16) return go(std::integral_constant<int, 16>());
        return go(std::integral_constant<int, 32>());
    });
}

// y: float32 dense [M, inner]; z: [M, inner] gate logits of the engine's type with row stride ldz; w: float32 [inner];
// out: dense [M, inner] of the engine's type.
extern "C" int ti_gate_group_rmsnorm(const float* y, const void* z, long long ldz, const float* w, void* out, int M, int inner,
                                     int groups, float eps, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && inner > 0 && groups > 0 && inner % groups == 0 && groups <= 65535, "gate_group_rmsnorm: %d channels in %d parts", inner, groups);
    const int gs = inner / groups;
    const int threads = gs <= 128 ? 64 : gs <= 1024 ? 128 : 256;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(gate_group_rmsnorm_kernel<T>, dim3(M, groups), dim3(threads), 0, stream, y, (const T*)z, ldz, w, (T*)out,
                                   inner, groups, eps));
        TI_CHECK_LAUNCH("gate_group_rmsnorm");
        return 0;
    });
}
