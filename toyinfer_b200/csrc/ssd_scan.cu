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
// Grid (column groups of 16, heads, sequences), 128 threads: a column's N values are shared out
// over 8 lanes (value n at lane n % 8), whose partial sums of y meet by three shuffles; B, C, x
// and the step sizes of a run of 16 tokens are staged in shared memory.
//
// gate_group_rmsnorm: v = y * silu(z);  v / rms(v) over each of `groups` equal parts of the row,
// times a weight per channel.
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int SCAN_THREADS = 128, LPC = 8, COLS = SCAN_THREADS / LPC, RUN = 16;

__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T, int R>
__global__ void __launch_bounds__(SCAN_THREADS)
ssd_scan_kernel(const T* __restrict__ xbc, long long ld_xbc, const T* __restrict__ dt_raw, long long ld_dt,
                const float* __restrict__ dt_bias, const float* __restrict__ rate, const float* __restrict__ skip,
                float* __restrict__ state, long long slot_stride, float* __restrict__ y, const int* __restrict__ cu_new,
                const int* __restrict__ seq_slot, int heads, int groups, int N, int vdim) {
    ti_pdl_trigger();
    constexpr int NP = LPC * R;                  // N rounded up to what the lanes hold
    extern __shared__ float sm[];
    float* Bs = sm;                              // [RUN][NP]
    float* Cs = Bs + RUN * NP;                   // [RUN][NP]
    float* xs = Cs + RUN * NP;                   // [RUN][COLS]
    float* ds = xs + RUN * COLS;                 // [RUN] step sizes
    float* as = ds + RUN;                        // [RUN] decays
    const int b = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, col = tid / LPC, sub = tid % LPC;
    const int v = v0 + col;
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const float hb = dt_bias[h], hr = rate[h], hd = skip ? skip[h] : 0.f;
    ti_pdl_sync();
    xbc = ti_dependent(xbc); dt_raw = ti_dependent(dt_raw);
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0) return;
    float* st = state + (size_t)seq_slot[b] * slot_stride + ((size_t)h * vdim + v) * N;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; r++) S[r] = (v < vdim && sub + LPC * r < N) ? st[sub + LPC * r] : 0.f;
    const T* Bg = xbc + inner + (size_t)g * N;
    const T* Cg = xbc + inner + (size_t)(groups + g) * N;
    for (int t0 = 0; t0 < n; t0 += RUN) {
        const int nt = min(RUN, n - t0);
        __syncthreads();        // the run before is used up
        for (int idx = tid; idx < nt * NP; idx += SCAN_THREADS) {
            const int t = idx / NP, j = idx - t * NP;
            const size_t at = (size_t)(tok0 + t0 + t) * ld_xbc;
            Bs[idx] = j < N ? to_f32(Bg[at + j]) : 0.f;
            Cs[idx] = j < N ? to_f32(Cg[at + j]) : 0.f;
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
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float a = as[t], xv = xs[t * COLS + col], dx = ds[t] * xv;
            const float* Bt = Bs + t * NP + sub;
            const float* Ct = Cs + t * NP + sub;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; r++) {
                S[r] = fmaf(a, S[r], dx * Bt[LPC * r]);
                acc = fmaf(S[r], Ct[LPC * r], acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (sub == 0 && v < vdim) y[(size_t)(tok0 + t0 + t) * inner + (size_t)h * vdim + v] = fmaf(hd, xv, acc);
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
        if (v < vdim && sub + LPC * r < N) st[sub + LPC * r] = S[r];
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
extern "C" int ti_ssd_scan(const void* xbc, long long ld_xbc, const void* dt_raw, long long ld_dt, const float* dt_bias,
                           const float* rate, const float* skip, float* state, long long slot_stride, float* y, const int* cu_new,
                           const int* seq_slot, int n_seq, int heads, int groups, int N, int vdim, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && heads > 0 && heads <= 65535 && groups > 0 && heads % groups == 0 && N > 0 && vdim > 0,
               "ssd_scan: bad sizes");
    TI_REQUIRE(N <= LPC * 32, "ssd_scan: a state of %d values per column is not supported (up to %d)", N, LPC * 32);
    const int rows = (N + LPC - 1) / LPC;
    dim3 grid((vdim + COLS - 1) / COLS, heads, n_seq);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto rv) -> int {
            constexpr int R = decltype(rv)::value;
            const size_t smem = ((size_t)2 * RUN * LPC * R + RUN * COLS + 2 * RUN) * sizeof(float);
            TI_CUDA(ti_launch(ssd_scan_kernel<T, R>, grid, dim3(SCAN_THREADS), smem, stream, (const T*)xbc, ld_xbc, (const T*)dt_raw, ld_dt,
                              dt_bias, rate, skip, state, slot_stride, y, cu_new, seq_slot, heads, groups, N, vdim));
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
