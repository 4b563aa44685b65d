// Several residual streams per token ("hyper-connections") kept in float32, and the norm that reads them.
//
// A token's state is X [S, H] (S streams of the model's width).  A sublayer f with the constants
// read a [S], carry C [S, S] (indexed [from, to]) and write b [S], and a per-channel scale g [H], does
//     u = sum_s a_s X_s;   y = g * f(norm(u));   X_t <- sum_s C_st X_s + b_t y   (all t from the old X).
// One kernel does what a sublayer boundary needs: the update that the sublayer BEFORE left pending
// (y of the engine's type, its g, C and b), written back to X, and the read of the sublayer AFTER
// (its a) with the RMS norm, y = u * rsqrt(mean(u^2) + eps) * w, rounded once into the engine's
// type.  With `rows` it works on the gathered rows only and leaves X alone (the head's rows; a = 1
// gives the sum of the streams).  S = 1 with C = b = a = 1 is a plain residual sum with a layer scale.
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int MAX_STREAMS = 8;

template <typename T, int S>
__global__ void hyper_norm_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ gain,
                                  const float* __restrict__ carry, const float* __restrict__ write,
                                  const float* __restrict__ read, const float* __restrict__ w, const int* __restrict__ rows,
                                  T* __restrict__ out, float* __restrict__ sum_out, int H, int M, float eps, int write_back) {
    ti_pdl_trigger();
    extern __shared__ float row[];      // H floats + 33
    float* red = row + H;
    __shared__ float c_s[S * S], b_s[S], a_s[S];
    if (threadIdx.x < S * S) c_s[threadIdx.x] = carry ? carry[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
    if (threadIdx.x < S) {
        b_s[threadIdx.x] = write ? write[threadIdx.x] : 1.f;
        a_s[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
    }
    ti_pdl_sync();
    X = ti_dependent(X); y = ti_dependent(y);
    __syncthreads();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    const bool ok = src >= 0 && src < M;
    if (!ok) src = 0;
    float* xr = X + (size_t)src * S * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x[S], xn[S];
#pragma unroll
        for (int s = 0; s < S; s++) x[s] = xr[(size_t)s * H + i];
        if (y) {
            const float yy = to_f32(y[(size_t)src * H + i]) * (gain ? gain[i] : 1.f);
#pragma unroll
            for (int t = 0; t < S; t++) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < S; s++) a = fmaf(c_s[s * S + t], x[s], a);
                xn[t] = fmaf(b_s[t], yy, a);
            }
            if (write_back) {
#pragma unroll
                for (int t = 0; t < S; t++) xr[(size_t)t * H + i] = xn[t];
            }
        } else {
#pragma unroll
            for (int t = 0; t < S; t++) xn[t] = x[t];
        }
        float u = 0.f;
#pragma unroll
        for (int t = 0; t < S; t++) u = fmaf(a_s[t], xn[t], u);
        if (!ok) u = 0.f;
        row[i] = u;
        if (sum_out) sum_out[(size_t)r * H + i] = u;
        ss = fmaf(u, u, ss);
    }
    if (!out) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)r * H + i] = from_f32<T>(w ? row[i] * inv * w[i] : row[i]);
}

}  // namespace

// X: float32 [M, S, H].  y: [M, H] of the engine's type or null (nothing pending).  gain: float32 [H] or null.
// carry [S * S], write [S], read [S]: float32 or null (identity, ones, ones).  w: float32 [H] norm weight, or
// null (`out` is the rounded u).  rows: null (every row, R == M) or R row indices.  out: [R, H] or null;
// sum_out: float32 [R, H] or null (u itself).  write_back: store the pending update into X.
extern "C" int ti_hyper_norm(float* X, const void* y, const float* gain, const float* carry, const float* write,
                             const float* read, const float* w, const int* rows, void* out, float* sum_out, int R, int H,
                             int M, int S, float eps, int write_back, int dtype, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && H > 0 && M > 0, "hyper_norm: bad sizes R=%d H=%d M=%d", R, H, M);
    TI_REQUIRE(S >= 1 && S <= MAX_STREAMS, "hyper_norm: %d streams are not supported (1 to %d)", S, MAX_STREAMS);
    TI_REQUIRE(rows || R == M, "hyper_norm: without row indices every row is taken (R=%d, M=%d)", R, M);
    TI_REQUIRE(!(rows && write_back), "hyper_norm: gathered rows are not written back");
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    TI_REQUIRE(smem <= 200 * 1024, "hyper_norm: rows of %d elements do not fit shared memory", H);
    // few rows (a step of single tokens): a block is alone on its SM and its time is a thread's chain of loads, so a row's
    // channels are spread over more threads
    const int threads = R <= 296 ? (H <= 256 ? 64 : H <= 512 ? 128 : H <= 1024 ? 256 : H <= 2048 ? 512 : 1024)
                                 : (H <= 256 ? 64 : H <= 1024 ? 128 : 256);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto sv) -> int {
            constexpr int SS = decltype(sv)::value;
            static size_t configured = 0;
            if (smem > 48 * 1024 && smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(hyper_norm_kernel<T, SS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch_class<1>(hyper_norm_kernel<T, SS>, dim3(R), dim3(threads), smem, stream, X, (const T*)y, gain, carry,
                                       write, read, w, rows, (T*)out, sum_out, H, M, eps, write_back));
            TI_CHECK_LAUNCH("hyper_norm");
            return 0;
        };
        switch (S) {
            case 1: return go(std::integral_constant<int, 1>());
            case 2: return go(std::integral_constant<int, 2>());
            case 3: return go(std::integral_constant<int, 3>());
            case 4: return go(std::integral_constant<int, 4>());
            case 5: return go(std::integral_constant<int, 5>());
            case 6: return go(std::integral_constant<int, 6>());
            case 7: return go(std::integral_constant<int, 7>());
            default: return go(std::integral_constant<int, 8>());
        }
    });
}
