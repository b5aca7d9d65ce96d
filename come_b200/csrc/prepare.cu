// Pre-attention preparation of the packed qkv tensor, one pass over q and k:
//   LayerNorm over the head dimension (q_norm / k_norm), 2-D rotary position embedding, and the per-key bias
//   log(count) -- everything the caller of the biased attention does between the qkv projection and the kernel.
// Also: integer positions of the packed rows straight from the merge plan (no feature-sized traffic).
//
// Bandwidth-bound: q and k are read and written once (v is never touched), 16 bytes per lane, several rows in
// flight per CTA.  The arithmetic follows the reference's sequence of roundings exactly (see the oracle).
#include <type_traits>

#include "come_internal.cuh"

namespace come {

constexpr int kPrepRowsInFlight = 4;
constexpr unsigned int kErrPositionRange = 1u << 16;  // a position indexed past the rotary tables

// 16-bit pair arithmetic with one rounding per operation and no fusing of a multiply into a following add.
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ float2 to_f32(T2 v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ T2 from_f32(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Pair<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ float2 to_f32(T2 v) { return __half22float2(v); }
    static __device__ __forceinline__ T2 from_f32(float a, float b) { return __floats2half2_rn(a, b); }
};

// Eight consecutive 16-bit features as four 32-bit words (one 16-byte access).
template <typename T> struct Vec8 {
    using T2 = typename Pair<T>::T2;
    uint32_t w[4];
    __device__ __forceinline__ T2 pair(int j) const { return *reinterpret_cast<const T2 *>(&w[j]); }
    __device__ __forceinline__ void set(int j, T2 v) { w[j] = *reinterpret_cast<const uint32_t *>(&v); }
    __device__ __forceinline__ void load(const T *src) {
        const uint4 v = *reinterpret_cast<const uint4 *>(src);
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    }
    __device__ __forceinline__ void load_ro(const T *src) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src));
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    }
    __device__ __forceinline__ void store(T *dst) const { *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]); }
    __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0u; }
};

// Sum over the `lanes` consecutive lanes that hold one head vector: butterfly, identical in every lane.
template <int LANES> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int m = 1; m < LANES; m <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// One CTA = 2 * H head vectors (q heads then k heads) x D/8 lanes; thread t owns 8 consecutive features of one head
// of q or of k for every row the CTA visits, so its gamma / beta stay in registers.
//
// Rounding sequence (identical to evaluating the reference's tensor expressions in the run dtype):
//   LayerNorm in float32: sums of x and of (x - mean)^2 in a fixed order (the squares accumulated with fused
//   multiply-adds), y = fma(gamma, rstd * (x - mean), beta), result rounded to T;
//   rotation: a = T(t * cos), b = T(rot(t) * sin), out = T(a + b).  Products of two 16-bit floats are exact in float32,
//   so the packed 16-bit multiply (one rounding) equals "multiply in float32, round to T"; likewise the packed add.
// Largest CTA the kernel is compiled for (64 registers per thread: four 256-thread CTAs per SM).
template <int D> constexpr int prep_max_threads() { return 512; }

template <typename T, int D, bool NORM, bool ROPE>
__global__ void __launch_bounds__(prep_max_threads<D>(), 2)
qkv_prepare_kernel(T *__restrict__ qkv, int total, int H, const T *__restrict__ q_gamma,
                   const T *__restrict__ q_beta, const T *__restrict__ k_gamma, const T *__restrict__ k_beta, float eps,
                   const int64_t *__restrict__ pos, const T *__restrict__ cos_t, const T *__restrict__ sin_t,
                   int table_rows, const float *__restrict__ weight, T *__restrict__ bias_out,
                   unsigned int *__restrict__ status) {
    using P2 = Pair<T>;
    constexpr int lanes = D >> 3;         // lanes per head vector (power of two, 4..32)
    const int hv = threadIdx.x / lanes;   // 0 .. 2H-1
    const int lane = threadIdx.x - hv * lanes;
    const int which = hv / H;             // 0 = q, 1 = k
    const int head = hv - which * H;
    const int feat = lane * 8;            // first feature of this lane inside the head
    constexpr int half = D >> 1;
    const int axis = feat >= half ? 1 : 0;   // y for the first half of the features, x for the second
    const int f_in_half = feat - axis * half;
    constexpr int partner = lanes >> 2;      // lane distance of the rotation partner (D/4 features)
    // second quarter of a half: rot = +t[f - D/4]; first quarter: rot = -t[f + D/4] (sign bits of both 16-bit halves)
    const uint32_t rot_sign = f_in_half >= (D >> 2) ? 0u : 0x80008000u;
    // 32-bit indexing in elements is safe: the host checks total * 3 * H * D < 2^31
    const int row_elems = 3 * H * D;
    const int col = which * H * D + head * D + feat;
    constexpr float inv_D = 1.0f / (float)D;  // D is a power of two: multiplying by 1/D rounds like dividing by D

    const T *gamma = which ? k_gamma : q_gamma;
    const T *beta = which ? k_beta : q_beta;
    f32x2_t g2[4], b2[4];  // this thread's 8 gamma / beta values as float32 pairs
#pragma unroll
    for (int j = 0; j < 4; ++j) g2[j] = b2[j] = 0ull;
    if constexpr (NORM) {
        Vec8<T> g, b;
        g.load(gamma + feat);
        b.load(beta + feat);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 gg = P2::to_f32(g.pair(j)), bb = P2::to_f32(b.pair(j));
            g2[j] = pack_f32x2(gg.x, gg.y);
            b2[j] = pack_f32x2(bb.x, bb.y);
        }
    }

    // Loads of one batch of kPrepRowsInFlight rows.  FULL batches (every row inside the tensor) carry no per-row
    // bounds checks; only the last batch of the tensor can be partial.
    auto load_batch = [&](auto full_tag, int r0, Vec8<T>(&x)[kPrepRowsInFlight], int(&p)[kPrepRowsInFlight]) {
        constexpr bool FULL = decltype(full_tag)::value;
#pragma unroll
        for (int i = 0; i < kPrepRowsInFlight; ++i) {
            const int r = r0 + i;
            p[i] = 0;
            if (FULL || r < total) {
                x[i].load(qkv + r * row_elems + col);
                if constexpr (ROPE) {
                    const int64_t pp = __ldg(pos + 2 * r + axis);
                    p[i] = (int)pp;
                    if ((uint64_t)pp >= (uint64_t)table_rows) {  // negative or past the table
                        if (hv == 0 && f_in_half == 0) atomicOr(status, kErrPositionRange);
                        p[i] = pp < 0 ? 0 : table_rows - 1;
                    }
                }
            } else {
                x[i].zero();
            }
        }
    };
    // Arithmetic and stores of one loaded batch.
    auto finish_batch = [&](auto full_tag, int r0, const Vec8<T>(&x)[kPrepRowsInFlight], const int(&p)[kPrepRowsInFlight]) {
        constexpr bool FULL = decltype(full_tag)::value;
#pragma unroll
        for (int i = 0; i < kPrepRowsInFlight; ++i) {
            const int r = r0 + i;
            const bool live = FULL || r < total;  // the whole CTA agrees: the shuffles below stay convergent
            Vec8<T> y = x[i];
            if constexpr (NORM) {
                // float32 pairs (f0,f1) (f2,f3) (f4,f5) (f6,f7): the even and the odd features are summed as two
                // left-to-right chains by packed adds, then added together
                f32x2_t v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 t = P2::to_f32(x[i].pair(j));
                    v[j] = pack_f32x2(t.x, t.y);
                }
                f32x2_t acc = add_f32x2(add_f32x2(add_f32x2(v[0], v[1]), v[2]), v[3]);
                float even, odd;
                unpack_f32x2(acc, even, odd);
                const float mean = __fmul_rn(group_sum<lanes>(__fadd_rn(even, odd)), inv_D);
                const f32x2_t neg_mean = pack_f32x2(-mean, -mean);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = add_f32x2(v[j], neg_mean);
                acc = mul_f32x2(v[0], v[0]);
#pragma unroll
                for (int j = 1; j < 4; ++j) acc = fma_f32x2(v[j], v[j], acc);  // explicit: never a separate mul + add
                unpack_f32x2(acc, even, odd);
                const float var = __fmul_rn(group_sum<lanes>(__fadd_rn(even, odd)), inv_D);
                const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
                const f32x2_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo, hi;
                    unpack_f32x2(fma_f32x2(g2[j], mul_f32x2(rstd2, v[j]), b2[j]), lo, hi);
                    y.set(j, P2::from_f32(lo, hi));
                }
            }
            if constexpr (ROPE) {
                Vec8<T> c, s, o;
                c.load_ro(cos_t + p[i] * half + f_in_half);
                s.load_ro(sin_t + p[i] * half + f_in_half);
#pragma unroll
                for (int j = 0; j < 4; ++j) o.w[j] = __shfl_xor_sync(0xffffffffu, y.w[j], partner) ^ rot_sign;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    y.set(j, __hadd2_rn(__hmul2_rn(y.pair(j), c.pair(j)), __hmul2_rn(o.pair(j), s.pair(j))));
            }
            if (live) {
                y.store(qkv + r * row_elems + col);
                if (bias_out && threadIdx.x == 0) bias_out[r] = Elem<T>::from_f32(logf(weight[r]));
            }
        }
    };

    // (Issuing the next batch's loads before the current batch's arithmetic was measured slower: the extra registers
    // cost a quarter of the resident warps.)
    const int full_end = total - total % kPrepRowsInFlight;  // rows covered by full batches
    Vec8<T> x[kPrepRowsInFlight];
    int p[kPrepRowsInFlight];
    int r0 = blockIdx.x * kPrepRowsInFlight;
    for (; r0 < full_end; r0 += gridDim.x * kPrepRowsInFlight) {
        load_batch(std::true_type{}, r0, x, p);
        finish_batch(std::true_type{}, r0, x, p);
    }
    if (r0 < total) {  // at most one CTA reaches the partial batch
        load_batch(std::false_type{}, r0, x, p);
        finish_batch(std::false_type{}, r0, x, p);
    }
}

// Positions of the packed rows of the image-token layout: special tokens (0, 0), patch (y, x) -> (y + 1, x + 1),
// merged window -> its centre.  One thread per source token; merged windows are written by their first token.
__global__ void packed_positions_kernel(const uint8_t *__restrict__ mask, const int64_t *__restrict__ rev_id,
                                        FrameLayout L, int64_t frames, int64_t *__restrict__ pos_out) {
    const int64_t total = frames * (int64_t)L.N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t bframe = i / L.N;
        const int n = (int)(i - bframe * L.N);
        int64_t y = 0, x = 0;
        bool write = true;
        if (n >= L.start) {
            const int p = n - L.start;
            const int py = p / L.W, px = p - py * L.W;
            y = py + 1;
            x = px + 1;
            if (py < L.Hc && px < L.Wc) {
                const int wy = py / L.gh, wx = px / L.gw;
                if (mask[bframe * L.M + (int64_t)wy * L.Wm + wx]) {
                    // mean of gh (gw) consecutive integers starting at wy*gh+1, in float like a merged bf16 tensor
                    // truncated to an integer: first + (g - 1) / 2 rounded toward zero after bf16 rounding
                    write = (py == wy * L.gh) && (px == wx * L.gw);
                    float sy = 0.0f, sx = 0.0f;
                    for (int a = 0; a < L.gh; ++a)
                        for (int c = 0; c < L.gw; ++c) {
                            sy = __fadd_rn(sy, __bfloat162float(__float2bfloat16_rn((float)(wy * L.gh + a + 1))));
                            sx = __fadd_rn(sx, __bfloat162float(__float2bfloat16_rn((float)(wx * L.gw + c + 1))));
                        }
                    const float G = (float)(L.gh * L.gw);
                    y = (int64_t)truncf(__bfloat162float(__float2bfloat16_rn(__fdiv_rn(sy, G))));
                    x = (int64_t)truncf(__bfloat162float(__float2bfloat16_rn(__fdiv_rn(sx, G))));
                }
            }
        }
        if (write) {
            const int64_t row = rev_id[i];
            pos_out[2 * row] = y;
            pos_out[2 * row + 1] = x;
        }
    }
}

template <typename T, int D, bool NORM, bool ROPE>
static int launch_prepare_k(void *qkv, int64_t total, int H, const void *qg, const void *qb, const void *kg,
                            const void *kb, float eps, const int64_t *pos, const void *cos_t, const void *sin_t,
                            int table_rows, const float *weight, void *bias_out, cudaStream_t st) {
    unsigned int *status = status_word_dev();
    if (!status) return COME_ERR_CUDA;
    const int threads = 2 * H * (D / 8);
    if (threads > prep_max_threads<D>() || threads % 32 != 0) {
        set_error("come_qkv_prepare: head_dim %d needs 2*num_heads*head_dim/8 = %d threads per row: must be a multiple of "
                  "32 and <= %d", D, threads, prep_max_threads<D>());
        return COME_ERR_UNSUPPORTED;
    }
    int resident = 0;  // CTAs of this size that fit one SM: the grid is exactly one resident wave
    COME_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, qkv_prepare_kernel<T, D, NORM, ROPE>, threads, 0));
    if (resident < 1) resident = 1;
    const int64_t iters = (total + kPrepRowsInFlight - 1) / kPrepRowsInFlight;
    const int64_t wave = (int64_t)sm_count() * resident;
    const unsigned grid = (unsigned)(iters < wave ? iters : wave);
    qkv_prepare_kernel<T, D, NORM, ROPE><<<grid, threads, 0, st>>>((T *)qkv, (int)total, H, (const T *)qg, (const T *)qb,
                                                      (const T *)kg, (const T *)kb, eps, pos, (const T *)cos_t,
                                                      (const T *)sin_t, table_rows, weight, (T *)bias_out, status);
    return check_launch("come_qkv_prepare");
}

template <typename T, int D>
static int launch_prepare_d(void *qkv, int64_t total, int H, const void *qg, const void *qb, const void *kg,
                            const void *kb, float eps, const int64_t *pos, const void *cos_t, const void *sin_t,
                            int table_rows, const float *weight, void *bias_out, cudaStream_t st) {
#define COME_PREP_ARGS qkv, total, H, qg, qb, kg, kb, eps, pos, cos_t, sin_t, table_rows, weight, bias_out, st
    if (qg && pos) return launch_prepare_k<T, D, true, true>(COME_PREP_ARGS);
    if (qg) return launch_prepare_k<T, D, true, false>(COME_PREP_ARGS);
    if (pos) return launch_prepare_k<T, D, false, true>(COME_PREP_ARGS);
    return launch_prepare_k<T, D, false, false>(COME_PREP_ARGS);  // only the bias is left to do
#undef COME_PREP_ARGS
}

template <typename T>
static int launch_prepare(void *qkv, int64_t total, int H, int D, const void *qg, const void *qb, const void *kg,
                          const void *kb, float eps, const int64_t *pos, const void *cos_t, const void *sin_t,
                          int table_rows, const float *weight, void *bias_out, cudaStream_t st) {
#define COME_PREP_CASE(DD) \
    case DD: return launch_prepare_d<T, DD>(qkv, total, H, qg, qb, kg, kb, eps, pos, cos_t, sin_t, table_rows, weight, bias_out, st)
    switch (D) {
        COME_PREP_CASE(32);
        COME_PREP_CASE(64);
        COME_PREP_CASE(128);
        COME_PREP_CASE(256);
    }
#undef COME_PREP_CASE
    set_error("come_qkv_prepare: unsupported head_dim %d", D);
    return COME_ERR_UNSUPPORTED;
}

}  // namespace come

using namespace come;

extern "C" int come_qkv_prepare(void *qkv_dev, int dtype, int64_t total, int num_heads, int head_dim,
                                const void *q_gamma_dev, const void *q_beta_dev, const void *k_gamma_dev,
                                const void *k_beta_dev, float eps, const int64_t *pos_dev, const void *cos_table_dev,
                                const void *sin_table_dev, int64_t table_rows, const float *weight_dev,
                                void *bias_out_dev, void *stream) {
    if (dtype == COME_F32) {
        set_error("come_qkv_prepare runs in the attention's dtype: float16 or bfloat16");
        return COME_ERR_UNSUPPORTED;
    }
    COME_REQUIRE(dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(total >= 0 && num_heads > 0 && head_dim > 0, "total must be >= 0, num_heads and head_dim > 0");
    if (!(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        set_error("come_qkv_prepare supports head_dim 32/64/128/256, got %d", head_dim);
        return COME_ERR_UNSUPPORTED;
    }
    COME_REQUIRE((q_gamma_dev == nullptr) == (q_beta_dev == nullptr) && (k_gamma_dev == nullptr) == (k_beta_dev == nullptr) &&
                     (q_gamma_dev == nullptr) == (k_gamma_dev == nullptr),
                 "q/k gamma and beta must be given together (all four) or not at all");
    COME_REQUIRE((weight_dev == nullptr) == (bias_out_dev == nullptr), "weight and bias_out must be given together");
    if (pos_dev) {
        COME_REQUIRE(cos_table_dev && sin_table_dev && table_rows > 0 && table_rows < (1ll << 31),
                     "positions need cos / sin tables with 0 < table_rows < 2^31");
        COME_REQUIRE((uintptr_t)cos_table_dev % 16 == 0 && (uintptr_t)sin_table_dev % 16 == 0,
                     "cos / sin tables must be 16-byte aligned");
    }
    if (total == 0) return COME_OK;
    COME_REQUIRE(total * 3 * (int64_t)num_heads * head_dim < (1ll << 31),
                 "come_qkv_prepare indexes with 32 bits: total * 3 * num_heads * head_dim must be < 2^31");
    COME_REQUIRE(qkv_dev != nullptr, "qkv must not be NULL");
    COME_REQUIRE((uintptr_t)qkv_dev % 16 == 0, "qkv must be 16-byte aligned");
    COME_REQUIRE(!q_gamma_dev || ((uintptr_t)q_gamma_dev % 16 == 0 && (uintptr_t)q_beta_dev % 16 == 0 &&
                                  (uintptr_t)k_gamma_dev % 16 == 0 && (uintptr_t)k_beta_dev % 16 == 0),
                 "gamma / beta must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == COME_BF16)
        return launch_prepare<__nv_bfloat16>(qkv_dev, total, num_heads, head_dim, q_gamma_dev, q_beta_dev, k_gamma_dev,
                                             k_beta_dev, eps, pos_dev, cos_table_dev, sin_table_dev, (int)table_rows,
                                             weight_dev, bias_out_dev, st);
    return launch_prepare<__half>(qkv_dev, total, num_heads, head_dim, q_gamma_dev, q_beta_dev, k_gamma_dev, k_beta_dev,
                                  eps, pos_dev, cos_table_dev, sin_table_dev, (int)table_rows, weight_dev, bias_out_dev, st);
}

extern "C" int come_packed_positions(const uint8_t *mask_dev, const int64_t *rev_id_dev, int64_t frames,
                                     const come_layout_t *layout, int64_t *pos_out_dev, void *stream) {
    FrameLayout L;
    int rc = make_layout(layout, &L);
    if (rc != COME_OK) return rc;
    COME_REQUIRE(L.H > 0, "come_packed_positions needs a 2-D layout (grid_h, grid_w > 0)");
    COME_REQUIRE(frames >= 0, "frames must be >= 0");
    if (frames == 0) return COME_OK;
    COME_REQUIRE(rev_id_dev && pos_out_dev && (L.M == 0 || mask_dev), "mask / rev_id / pos_out must not be NULL");
    const int64_t total = frames * (int64_t)L.N;
    const int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    packed_positions_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, (cudaStream_t)stream>>>(
        mask_dev, rev_id_dev, L, frames, pos_out_dev);
    return check_launch("come_packed_positions");
}
