// Confidence-guided window selection for sm_100a: window means, quantile threshold, boolean merge mask.
//
// One CTA owns one quantile group (all windows of a batch element, or of one frame).  The window means are
// built in shared memory, sorted there with a bitonic network, the two order statistics around the requested
// rank are interpolated exactly like torch.quantile does, and the mask is written from freshly recomputed
// means (the arithmetic is deterministic, so the recomputed value equals the sorted one bit for bit).
#include "come_internal.cuh"

namespace come {

constexpr int kSelectThreads = 512;
constexpr int kSelectMaxWindows = 32768;

template <typename T> __device__ __forceinline__ float round_store(float x) { return Elem<T>::to_f32(Elem<T>::from_f32(x)); }
template <typename T> static float dtype_round_host(float x);
template <> float dtype_round_host<float>(float x) { return x; }
template <> float dtype_round_host<__half>(float x) { return __half2float(__float2half_rn(x)); }
template <> float dtype_round_host<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Mean confidence of window m of frame f: float32 sum over the window row by row, divided by its size,
// rounded to the confidence dtype (a tensor of that dtype holds the mean in the reference).
template <typename T>
__device__ __forceinline__ float window_mean(const T *__restrict__ conf, int64_t f, int m, int H, int W, int gh,
                                             int gw, int Wm) {
    const int wy = m / Wm, wx = m - wy * Wm;
    const T *p = conf + f * (int64_t)H * W + (int64_t)(wy * gh) * W + wx * gw;
    float acc = 0.0f;
    for (int iy = 0; iy < gh; ++iy)
        for (int ix = 0; ix < gw; ++ix) acc = __fadd_rn(acc, Elem<T>::to_f32(p[iy * W + ix]));
    return round_store<T>(__fdiv_rn(acc, (float)(gh * gw)));
}

template <typename T>
__global__ void __launch_bounds__(kSelectThreads)
select_rank_kernel(const T *__restrict__ conf, int frames_per_group, int H, int W, int gh, int gw, float q_all,
                   const float *__restrict__ q_per_group, uint8_t *__restrict__ mask) {
    const float q = q_per_group ? fminf(fmaxf(q_per_group[blockIdx.x], 0.0f), 1.0f) : q_all;
    extern __shared__ float s_val[];  // n_pow2 floats
    __shared__ float s_thr;
    const int Wm = W / gw, M = (H / gh) * Wm;
    const int n = frames_per_group * M;
    int n_pow2 = 1;
    while (n_pow2 < n) n_pow2 <<= 1;
    const int64_t f0 = (int64_t)blockIdx.x * frames_per_group;

    for (int i = threadIdx.x; i < n_pow2; i += kSelectThreads) {
        float v = __int_as_float(0x7f800000);  // +inf padding sorts to the end
        if (i < n) v = window_mean<T>(conf, f0 + i / M, i % M, H, W, gh, gw, Wm);
        s_val[i] = v;
    }
    __syncthreads();
    for (int k = 2; k <= n_pow2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pow2; i += kSelectThreads) {
                const int partner = i ^ j;
                if (partner > i) {
                    const float a = s_val[i], b = s_val[partner];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) {
                        s_val[i] = b;
                        s_val[partner] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
    if (threadIdx.x == 0) {
        // torch.quantile, linear interpolation: rank = q * (n - 1) in float32; fused lerp that switches
        // formula at weight 0.5 (fma(w, d, a) below, fma(w - 1, d, b) from there on)
        const float rank = __fmul_rn(q, (float)(n - 1));
        const float lo = floorf(rank), hi = ceilf(rank);
        const float w = __fsub_rn(rank, lo);
        const float a = s_val[(int)lo], b = s_val[(int)hi];
        const float d = __fsub_rn(b, a);
        s_thr = (w < 0.5f) ? __fmaf_rn(w, d, a) : __fmaf_rn(__fsub_rn(w, 1.0f), d, b);
    }
    __syncthreads();
    const float thr = s_thr;
    for (int i = threadIdx.x; i < n; i += kSelectThreads) {
        const float v = window_mean<T>(conf, f0 + i / M, i % M, H, W, gh, gw, Wm);
        mask[f0 * M + i] = v < thr ? 1 : 0;
    }
}

template <typename T>
__global__ void select_abs_kernel(const T *__restrict__ conf, int64_t n_windows, int H, int W, int gh, int gw,
                                  float thr, uint8_t *__restrict__ mask) {
    const int Wm = W / gw, M = (H / gh) * Wm;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_windows; i += (int64_t)gridDim.x * blockDim.x)
        mask[i] = window_mean<T>(conf, i / M, (int)(i % M), H, W, gh, gw, Wm) < thr ? 1 : 0;  // thr already rounded to T
}

// Block-wide sum of doubles (every thread returns the total).  `scratch` holds one double per warp.
__device__ __forceinline__ double block_sum_f64(double v, double *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    __syncthreads();  // scratch may still be read by the previous call
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < kSelectThreads / 32; ++w) total += scratch[w];
    return total;
}

// Z-normalised selection (the reference's "mse" confidence mode): per batch element, x -> (x - mean) / (std + 1e-3) with
// the unbiased standard deviation, then the window mean of the normalised values against the threshold.  Every tensor
// operation of the reference's expression rounds to the confidence dtype; mean and variance are accumulated in float64.
// One CTA per batch element.
template <typename T>
__global__ void __launch_bounds__(kSelectThreads)
select_zscore_kernel(const T *__restrict__ conf, int frames_per_batch, int H, int W, int gh, int gw, float thr,
                     uint8_t *__restrict__ mask) {
    __shared__ double s_part[kSelectThreads / 32];
    const int Wm = W / gw, M = (H / gh) * Wm;
    const int64_t n = (int64_t)frames_per_batch * H * W;
    const T *x = conf + (int64_t)blockIdx.x * n;
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < n; i += kSelectThreads) acc += (double)Elem<T>::to_f32(x[i]);
    const double mean64 = block_sum_f64(acc, s_part) / (double)n;
    acc = 0.0;
    for (int64_t i = threadIdx.x; i < n; i += kSelectThreads) {
        const double d = (double)Elem<T>::to_f32(x[i]) - mean64;
        acc += d * d;
    }
    const double var64 = block_sum_f64(acc, s_part) / (double)(n - 1);  // n == 1: 0 / 0 = NaN, nothing is merged
    const float mean = round_store<T>((float)mean64);
    const float sd = round_store<T>((float)sqrt(var64));
    const float den = round_store<T>(__fadd_rn(sd, 1e-3f));
    const float thr_t = round_store<T>(thr);  // a tensor compared with a number: the number is rounded to the tensor's dtype
    const int64_t f0 = (int64_t)blockIdx.x * frames_per_batch;
    for (int i = threadIdx.x; i < frames_per_batch * M; i += kSelectThreads) {
        const int f = i / M, m = i - f * M;
        const int wy = m / Wm, wx = m - wy * Wm;
        const T *p = x + (int64_t)f * H * W + (int64_t)(wy * gh) * W + wx * gw;
        float sum = 0.0f;
        for (int iy = 0; iy < gh; ++iy)
            for (int ix = 0; ix < gw; ++ix) {
                const float c = round_store<T>(__fsub_rn(Elem<T>::to_f32(p[iy * W + ix]), mean));
                sum = __fadd_rn(sum, round_store<T>(__fdiv_rn(c, den)));
            }
        const float v = round_store<T>(__fdiv_rn(sum, (float)(gh * gw)));
        mask[f0 * M + i] = v < thr_t ? 1 : 0;
    }
}

template <typename T>
static int launch_select(const void *conf, int64_t batch, int64_t S, int H, int W, int gh, int gw, float thr,
                         const float *thr_per_group, int mode, int scope, uint8_t *mask, cudaStream_t st) {
    const int M = (H / gh) * (W / gw);
    if (mode == COME_SELECT_ABS) {
        const int64_t n = batch * S * M;
        int64_t blocks = (n + 255) / 256;
        if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
        // a tensor compared with a Python number: the number is first rounded to the tensor's dtype
        const float thr_t = dtype_round_host<T>(thr);
        select_abs_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T *)conf, n, H, W, gh, gw, thr_t, mask);
        return check_launch("come_select_windows");
    }
    if (mode == COME_SELECT_ZSCORE) {
        select_zscore_kernel<T><<<(unsigned)batch, kSelectThreads, 0, st>>>((const T *)conf, (int)S, H, W, gh, gw, thr, mask);
        return check_launch("come_select_windows");
    }
    const int64_t groups = scope == COME_SCOPE_BATCH ? batch : batch * S;
    const int frames_per_group = scope == COME_SCOPE_BATCH ? (int)S : 1;
    const int64_t n = (int64_t)frames_per_group * M;
    COME_REQUIRE(n <= kSelectMaxWindows, "at most %d windows per quantile group, got %lld", kSelectMaxWindows, (long long)n);
    int n_pow2 = 1;
    while (n_pow2 < n) n_pow2 <<= 1;
    const size_t smem = (size_t)n_pow2 * sizeof(float);
    if (smem > 48 * 1024)
        COME_CUDA(cudaFuncSetAttribute(select_rank_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSelectMaxWindows * (int)sizeof(float)));
    select_rank_kernel<T><<<(unsigned)groups, kSelectThreads, smem, st>>>((const T *)conf, frames_per_group, H, W, gh, gw,
                                                                          thr, thr_per_group, mask);
    return check_launch("come_select_windows");
}

}  // namespace come

using namespace come;

static int select_impl(const void *conf_dev, int dtype, int64_t batch, int64_t frames_per_batch, int grid_h, int grid_w,
                       int group_h, int group_w, float threshold, const float *thr_per_group, int mode, int scope,
                       uint8_t *mask_dev, void *stream) {
    COME_REQUIRE(batch >= 0 && frames_per_batch >= 0, "batch and frames_per_batch must be >= 0");
    COME_REQUIRE(grid_h > 0 && grid_w > 0 && group_h > 0 && group_w > 0, "grid and window sizes must be positive");
    COME_REQUIRE(group_h <= grid_h && group_w <= grid_w, "window larger than the grid");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(mode == COME_SELECT_RANK || mode == COME_SELECT_ABS || mode == COME_SELECT_ZSCORE, "unknown selection mode %d", mode);
    COME_REQUIRE(frames_per_batch * (int64_t)grid_h * grid_w < (1ll << 31), "a batch element holds too many confidences");
    COME_REQUIRE(scope == COME_SCOPE_BATCH || scope == COME_SCOPE_FRAME, "unknown selection scope %d", scope);
    COME_REQUIRE(thr_per_group == nullptr || mode == COME_SELECT_RANK, "per-group thresholds need the ranking mode");
    if (mode == COME_SELECT_RANK && !thr_per_group)
        COME_REQUIRE(threshold >= 0.0f && threshold <= 1.0f, "Ranking mode requires threshold in [0, 1], got %g", threshold);
    if (batch == 0 || frames_per_batch == 0) return COME_OK;
    COME_REQUIRE(conf_dev && mask_dev, "conf / mask must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case COME_F32: return launch_select<float>(conf_dev, batch, frames_per_batch, grid_h, grid_w, group_h, group_w, threshold, thr_per_group, mode, scope, mask_dev, st);
        case COME_F16: return launch_select<__half>(conf_dev, batch, frames_per_batch, grid_h, grid_w, group_h, group_w, threshold, thr_per_group, mode, scope, mask_dev, st);
        default: return launch_select<__nv_bfloat16>(conf_dev, batch, frames_per_batch, grid_h, grid_w, group_h, group_w, threshold, thr_per_group, mode, scope, mask_dev, st);
    }
}

extern "C" int come_select_windows(const void *conf_dev, int dtype, int64_t batch, int64_t frames_per_batch,
                                   int grid_h, int grid_w, int group_h, int group_w, float threshold, int mode,
                                   int scope, uint8_t *mask_dev, void *stream) {
    return select_impl(conf_dev, dtype, batch, frames_per_batch, grid_h, grid_w, group_h, group_w, threshold, nullptr, mode,
                       scope, mask_dev, stream);
}

extern "C" int come_select_windows_ratios(const void *conf_dev, int dtype, int64_t batch, int64_t frames_per_batch,
                                          int grid_h, int grid_w, int group_h, int group_w, const float *ratios_dev,
                                          int scope, uint8_t *mask_dev, void *stream) {
    COME_REQUIRE(ratios_dev != nullptr, "ratios must not be NULL");
    return select_impl(conf_dev, dtype, batch, frames_per_batch, grid_h, grid_w, group_h, group_w, 0.5f, ratios_dev,
                       COME_SELECT_RANK, scope, mask_dev, stream);
}
