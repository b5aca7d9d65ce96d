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
        mask[i] = window_mean<T>(conf, i / M, (int)(i % M), H, W, gh, gw, Wm) < thr ? 1 : 0;
}

template <typename T>
static int launch_select(const void *conf, int64_t batch, int64_t S, int H, int W, int gh, int gw, float thr,
                         const float *thr_per_group, int mode, int scope, uint8_t *mask, cudaStream_t st) {
    const int M = (H / gh) * (W / gw);
    if (mode == COME_SELECT_ABS) {
        const int64_t n = batch * S * M;
        int64_t blocks = (n + 255) / 256;
        if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
        select_abs_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T *)conf, n, H, W, gh, gw, thr, mask);
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
    COME_REQUIRE(mode == COME_SELECT_RANK || mode == COME_SELECT_ABS, "unknown selection mode %d", mode);
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
