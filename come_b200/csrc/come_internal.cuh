// Shared helpers of the come_b200 CUDA sources: error reporting, dtype traits, the frame layout.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/come_b200.h"

namespace come {

// ---- host-side error reporting ---------------------------------------------------------------------------
void set_error(const char *fmt, ...);

#define COME_REQUIRE(cond, ...)          \
    do {                                 \
        if (!(cond)) {                   \
            ::come::set_error(__VA_ARGS__); \
            return COME_ERR_ARG;         \
        }                                \
    } while (0)

#define COME_CUDA(call)                                                                      \
    do {                                                                                     \
        cudaError_t e__ = (call);                                                            \
        if (e__ != cudaSuccess) {                                                            \
            ::come::set_error("%s failed: %s", #call, cudaGetErrorString(e__));              \
            return COME_ERR_CUDA;                                                            \
        }                                                                                    \
    } while (0)

inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: kernel launch failed: %s", what, cudaGetErrorString(e));
        return COME_ERR_CUDA;
    }
    return COME_OK;
}

inline size_t dtype_size(int dtype) { return dtype == COME_F32 ? 4 : 2; }

// Number of SMs of the current device (cached per device).
int sm_count();

// ---- device status word -----------------------------------------------------------------------------------
// Address of the library's device status word on the current device (NULL and an error message on failure).
unsigned int *status_word_dev();

// ---- element conversion -------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f32(float x) { return x; }
    static __device__ __forceinline__ float from_f32(float x) { return x; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};

// ---- packed float32x2 arithmetic (sm_100: one instruction for two lanes, each rounded to nearest like the scalar op) --
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack_f32x2(float lo, float hi) {
    f32x2_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack_f32x2(f32x2_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t fma_f32x2(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2_t add_f32x2(f32x2_t a, f32x2_t b) {
    f32x2_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2_t mul_f32x2(f32x2_t a, f32x2_t b) {
    f32x2_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// ---- frame layout (device view of come_layout_t) -------------------------------------------------------------
struct FrameLayout {
    int start;     // special tokens
    int H, W;      // patch grid (H == 0: 1-D operator)
    int gh, gw;    // window
    int Wm;        // windows per grid row
    int Hc, Wc;    // extent covered by windows
    int edge_cols; // W - Wc
    int prefix;    // never-merged rows of a frame: specials + uncovered patches
    int G;         // tokens per group
    int M;         // groups per frame
    int N;         // tokens per frame

    // merge-order row r of a frame (prefix rows, then M groups of G rows) -> token index inside the frame
    __host__ __device__ __forceinline__ int src_token(int r) const {
        if (H == 0 || r < start) return r;
        if (r < prefix) {
            int e = r - start;
            int n_right = Hc * edge_cols;
            int y, x;
            if (e < n_right) {
                y = e / edge_cols;
                x = Wc + e % edge_cols;
            } else {
                e -= n_right;
                y = Hc + e / W;
                x = e % W;
            }
            return start + y * W + x;
        }
        r -= prefix;
        int m = r / G, g = r - m * G;
        int wy = m / Wm, wx = m - wy * Wm;
        int iy = g / gw, ix = g - iy * gw;
        return start + (wy * gh + iy) * W + wx * gw + ix;
    }
};

// Validates a come_layout_t and expands it; returns COME_OK or COME_ERR_ARG (message set).
int make_layout(const come_layout_t *in, FrameLayout *out);

}  // namespace come
