// Variable-length biased attention forward: argument checking, dispatch, and the CUDA-core kernel that
// serves every head dimension the tensor-core kernel does not (anything but 64).
#include "come_internal.cuh"
#include "attn_sm100.cuh"

namespace come {

constexpr int kGenericWarps = 4;
constexpr int kGenericMaxD = 256;

// One warp per query row.  Lanes split the keys 32 at a time for the scores and split the head dimension
// for the output accumulation; softmax statistics are kept online in float32.
template <typename T>
__global__ void __launch_bounds__(kGenericWarps * 32)
attn_generic_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, int64_t q_rs,
                    int64_t k_rs, int64_t v_rs, const T *__restrict__ bias, const int *__restrict__ cu, int H, int D,
                    float scale, T *__restrict__ out, int64_t o_rs, float *__restrict__ lse, int q_begin, int q_end,
                    int kv_total, int q_free) {
    __shared__ float s_q[kGenericWarps][kGenericMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = blockIdx.y, h = blockIdx.z;
    const int s0 = cu ? cu[seg] : 0, s1 = cu ? cu[seg + 1] : kv_total;
    // global row; q / out / lse hold rows [q_begin, q_end).  q_free: one segment that every query row attends to
    const int row = (q_free ? q_begin : max(s0, q_begin)) + blockIdx.x * kGenericWarps + warp;
    if (row >= (q_free ? q_end : min(s1, q_end))) return;  // whole warp leaves together

    const T *qrow = q + (int64_t)(row - q_begin) * q_rs + (int64_t)h * D;
    for (int d = lane; d < D; d += 32) s_q[warp][d] = Elem<T>::to_f32(qrow[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[kGenericMaxD / 32];
#pragma unroll
    for (int i = 0; i < kGenericMaxD / 32; ++i) acc[i] = 0.0f;

    for (int j0 = s0; j0 < s1; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j < s1) {
            const T *krow = k + (int64_t)j * k_rs + (int64_t)h * D;
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot = fmaf(s_q[warp][d], Elem<T>::to_f32(krow[d]), dot);
            s = dot * scale + (bias ? Elem<T>::to_f32(bias[j]) : 0.0f);
        }
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m, mx);
        const float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        const float p = (j < s1 && m_new != -INFINITY) ? expf(s - m_new) : 0.0f;
        float psum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * alpha + psum;
#pragma unroll
        for (int i = 0; i < kGenericMaxD / 32; ++i) acc[i] *= alpha;
        const int nk = min(32, s1 - j0);
        for (int t = 0; t < nk; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const T *vrow = v + (int64_t)(j0 + t) * v_rs + (int64_t)h * D;
#pragma unroll
            for (int i = 0; i < kGenericMaxD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pt, Elem<T>::to_f32(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
    T *orow = out + (int64_t)(row - q_begin) * o_rs + (int64_t)h * D;
#pragma unroll
    for (int i = 0; i < kGenericMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = Elem<T>::from_f32(acc[i] * inv);
    }
    if (lse && lane == 0) lse[(int64_t)h * (q_end - q_begin) + (row - q_begin)] = m + logf(l);
}

template <typename T>
static int launch_generic(const void *q, const void *k, const void *v, int64_t q_rs, int64_t k_rs, int64_t v_rs,
                          const void *bias, const int *cu, int nseg, int max_seqlen, int H, int D, float scale, void *out,
                          int64_t o_rs, float *lse, int64_t q_begin, int64_t q_end, int64_t kv_total, bool q_free, cudaStream_t st) {
    const int64_t span = (!q_free && max_seqlen < q_end - q_begin) ? max_seqlen : q_end - q_begin;
    dim3 grid((unsigned)((span + kGenericWarps - 1) / kGenericWarps), nseg, H);
    attn_generic_kernel<T><<<grid, kGenericWarps * 32, 0, st>>>((const T *)q, (const T *)k, (const T *)v, q_rs, k_rs, v_rs,
                                                                (const T *)bias, cu, H, D, scale, (T *)out, o_rs, lse, (int)q_begin, (int)q_end,
                                                                (int)kv_total, q_free ? 1 : 0);
    return check_launch("come_attn_varlen_fwd (CUDA-core kernel)");
}

// out = (w_a * out_a + w_b * out_b) / (w_a + w_b) with w_x = exp(lse_x - max(lse_a, lse_b)): the exact merge of two
// attention results over disjoint key sets.  A thread owns 8 consecutive features (16 bytes) of a (row, head).
template <typename T>
__global__ void __launch_bounds__(256)
attn_combine_kernel(const T *__restrict__ oa, const float *__restrict__ la, const T *__restrict__ ob,
                    const float *__restrict__ lb, int64_t rows, int H, int D, T *__restrict__ out, float *__restrict__ lse_out) {
    const int per_head = D / 8;
    const int64_t n = rows * H * per_head;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t rh = i / per_head;  // row * H + head
        const int64_t row = rh / H;
        const int h = (int)(rh - row * H);
        const float a = la[(int64_t)h * rows + row], b = lb[(int64_t)h * rows + row];
        const float m = fmaxf(a, b);
        float wa = 0.0f, wb = 0.0f, inv = 0.0f;
        if (m > -INFINITY) {  // both key sets empty: the row stays zero
            wa = expf(a - m);
            wb = expf(b - m);
            inv = 1.0f / (wa + wb);
        }
        const uint4 va = reinterpret_cast<const uint4 *>(oa)[i], vb = reinterpret_cast<const uint4 *>(ob)[i];
        const T *xa = reinterpret_cast<const T *>(&va), *xb = reinterpret_cast<const T *>(&vb);
        uint4 vo;
        T *xo = reinterpret_cast<T *>(&vo);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            xo[e] = Elem<T>::from_f32((wa * Elem<T>::to_f32(xa[e]) + wb * Elem<T>::to_f32(xb[e])) * inv);
        reinterpret_cast<uint4 *>(out)[i] = vo;
        if (lse_out && (i - rh * per_head) == 0) lse_out[(int64_t)h * rows + row] = (m > -INFINITY) ? m + logf(wa + wb) : -INFINITY;
    }
}

// The same merge for `parts` results stored one behind the other (out_p = parts_out + p * part_o elements,
// lse_p = parts_lse + p * H * rows floats): the shares of a launch that split the keys of its work items.
template <typename T>
__global__ void __launch_bounds__(256)
attn_combine_parts_kernel(const T *__restrict__ parts_out, const float *__restrict__ parts_lse, int parts, int64_t part_o,
                          int64_t rows, int H, int D, T *__restrict__ out, float *__restrict__ lse_out) {
    const int per_head = D / 8;
    const int64_t n = rows * H * per_head;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t rh = i / per_head;
        const int64_t row = rh / H;
        const int h = (int)(rh - row * H);
        const int64_t l_at = (int64_t)h * rows + row;
        float m = -INFINITY;
        for (int p = 0; p < parts; ++p) m = fmaxf(m, parts_lse[(int64_t)p * H * rows + l_at]);
        float acc[8] = {}, wsum = 0.0f;
        if (m > -INFINITY) {
            for (int p = 0; p < parts; ++p) {
                const float w = expf(parts_lse[(int64_t)p * H * rows + l_at] - m);
                const uint4 v = reinterpret_cast<const uint4 *>(parts_out + (int64_t)p * part_o)[i];
                const T *x = reinterpret_cast<const T *>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += w * Elem<T>::to_f32(x[e]);
                wsum += w;
            }
        }
        const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
        uint4 vo;
        T *xo = reinterpret_cast<T *>(&vo);
#pragma unroll
        for (int e = 0; e < 8; ++e) xo[e] = Elem<T>::from_f32(acc[e] * inv);
        reinterpret_cast<uint4 *>(out)[i] = vo;
        if (lse_out && (i - rh * per_head) == 0) lse_out[l_at] = (m > -INFINITY) ? m + logf(wsum) : -INFINITY;
    }
}

}  // namespace come

using namespace come;

static int attn_dispatch(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t total,
                         int64_t q_begin, int64_t q_rows, int num_heads, int head_dim, int64_t q_row_stride,
                         int64_t k_row_stride, int64_t v_row_stride, const void *bias_dev, const int32_t *cu_seqlens_dev,
                         int num_segments, int max_seqlen, const int32_t *max_seqlen_dev, float softmax_scale, void *out_dev,
                         int64_t out_row_stride, float *lse_dev, int backend, void *stream, bool q_free = false, int k_parts = 1,
                         int64_t part_o = 0) {
    COME_REQUIRE(dtype == COME_F16 || dtype == COME_BF16, "FlashAttention only support fp16 and bf16 data type");
    COME_REQUIRE(num_segments > 0, "batch size must be positive");
    COME_REQUIRE(total >= 0 && num_heads > 0, "total must be >= 0 and num_heads > 0");
    COME_REQUIRE(q_begin >= 0 && q_rows >= 0 && (q_free || q_begin + q_rows <= total), "query rows [%lld, %lld) must lie inside [0, %lld)",
                 (long long)q_begin, (long long)(q_begin + q_rows), (long long)total);
    COME_REQUIRE(q_rows < (1ll << 31), "query rows must fit int32");
    COME_REQUIRE(head_dim > 0 && head_dim <= 256, "FlashAttention forward only supports head dimension at most 256");
    COME_REQUIRE(head_dim % 8 == 0, "query, key, value, and out_ must have a head_size that is a multiple of 8");
    COME_REQUIRE(max_seqlen >= 0, "max_seqlen must be >= 0");
    COME_REQUIRE(backend >= 0 && backend <= 2, "unknown backend %d", backend);
    const int64_t hd = (int64_t)num_heads * head_dim;
    COME_REQUIRE(q_row_stride >= hd && k_row_stride >= hd && v_row_stride >= hd && out_row_stride >= hd,
                 "row strides must cover num_heads * head_dim elements");
    COME_REQUIRE(total < (1ll << 31), "total tokens must fit int32");
    if (total == 0 || max_seqlen == 0 || q_rows == 0) return COME_OK;
    COME_REQUIRE(q_dev && k_dev && v_dev && out_dev && (cu_seqlens_dev || q_free), "q / k / v / out / cu_seqlens must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;

    AttnArgs a;
    a.q = q_dev; a.k = k_dev; a.v = v_dev; a.bias = bias_dev; a.cu = cu_seqlens_dev; a.out = out_dev; a.lse = lse_dev;
    a.dtype = dtype; a.total = total; a.q_begin = q_begin; a.q_end = q_begin + q_rows; a.H = num_heads; a.D = head_dim;
    a.q_rs = q_row_stride; a.k_rs = k_row_stride; a.v_rs = v_row_stride; a.o_rs = out_row_stride;
    a.nseg = num_segments; a.max_seqlen = max_seqlen; a.max_seqlen_dev = max_seqlen_dev; a.scale = softmax_scale;
    a.q_free = q_free;
    a.k_parts = k_parts;
    a.part_o = part_o;
    a.part_l = (int64_t)num_heads * q_rows;

    const bool tc_ok = attn_sm100_supported(a);
    if (backend == 2 && !tc_ok) {
        set_error("tcgen05 attention needs head_dim 64, a positive scale, 16-byte aligned q/k/v/out and strides that are multiples of 8 elements");
        return COME_ERR_UNSUPPORTED;
    }
    if (tc_ok && backend != 1) return attn_sm100_launch(a, st);
    if (k_parts > 1) {
        set_error("attention with key shares runs on the tcgen05 kernel only (head_dim 64, TMA-compatible tensors, backend auto or tcgen05)");
        return COME_ERR_UNSUPPORTED;
    }
    if (dtype == COME_F16)
        return launch_generic<__half>(q_dev, k_dev, v_dev, q_row_stride, k_row_stride, v_row_stride, bias_dev, cu_seqlens_dev,
                                      num_segments, max_seqlen, num_heads, head_dim, softmax_scale, out_dev, out_row_stride,
                                      lse_dev, a.q_begin, a.q_end, total, q_free, st);
    return launch_generic<__nv_bfloat16>(q_dev, k_dev, v_dev, q_row_stride, k_row_stride, v_row_stride, bias_dev,
                                         cu_seqlens_dev, num_segments, max_seqlen, num_heads, head_dim, softmax_scale,
                                         out_dev, out_row_stride, lse_dev, a.q_begin, a.q_end, total, q_free, st);
}

extern "C" int come_attn_varlen_fwd(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t total,
                                    int num_heads, int head_dim, int64_t q_row_stride, int64_t k_row_stride,
                                    int64_t v_row_stride, const void *bias_dev, const int32_t *cu_seqlens_dev,
                                    int num_segments, int max_seqlen, float softmax_scale, void *out_dev,
                                    int64_t out_row_stride, float *lse_dev, int backend, void *stream) {
    return attn_dispatch(q_dev, k_dev, v_dev, dtype, total, 0, total, num_heads, head_dim, q_row_stride, k_row_stride,
                         v_row_stride, bias_dev, cu_seqlens_dev, num_segments, max_seqlen, nullptr, softmax_scale, out_dev,
                         out_row_stride, lse_dev, backend, stream);
}

extern "C" int come_attn_varlen_fwd_rows(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t total,
                                         int64_t q_row_begin, int64_t q_rows, int num_heads, int head_dim,
                                         int64_t q_row_stride, int64_t k_row_stride, int64_t v_row_stride,
                                         const void *bias_dev, const int32_t *cu_seqlens_dev, int num_segments,
                                         int max_seqlen, const int32_t *max_seqlen_dev, float softmax_scale, void *out_dev,
                                         int64_t out_row_stride, float *lse_dev, int backend, void *stream) {
    return attn_dispatch(q_dev, k_dev, v_dev, dtype, total, q_row_begin, q_rows, num_heads, head_dim, q_row_stride,
                         k_row_stride, v_row_stride, bias_dev, cu_seqlens_dev, num_segments, max_seqlen, max_seqlen_dev,
                         softmax_scale, out_dev, out_row_stride, lse_dev, backend, stream);
}


extern "C" int come_attn_cross_fwd(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t q_rows,
                                   int64_t kv_rows, int num_heads, int head_dim, int64_t q_row_stride, int64_t k_row_stride,
                                   int64_t v_row_stride, const void *bias_dev, float softmax_scale, void *out_dev,
                                   int64_t out_row_stride, float *lse_dev, int backend, void *stream) {
    COME_REQUIRE(kv_rows > 0 || q_rows == 0, "come_attn_cross_fwd needs at least one key");
    const int max_len = (int)(kv_rows < (1ll << 31) ? kv_rows : 0);
    return attn_dispatch(q_dev, k_dev, v_dev, dtype, kv_rows, 0, q_rows, num_heads, head_dim, q_row_stride, k_row_stride,
                         v_row_stride, bias_dev, nullptr, 1, max_len, nullptr, softmax_scale, out_dev, out_row_stride,
                         lse_dev, backend, stream, true);
}

extern "C" int come_attn_cross_fwd_parts(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t q_rows,
                                         int64_t kv_rows, int num_heads, int head_dim, int64_t q_row_stride,
                                         int64_t k_row_stride, int64_t v_row_stride, const void *bias_dev, float softmax_scale,
                                         int key_parts, void *out_parts_dev, float *lse_parts_dev, int backend, void *stream) {
    COME_REQUIRE(kv_rows > 0 || q_rows == 0, "come_attn_cross_fwd_parts needs at least one key");
    COME_REQUIRE(key_parts >= 1 && key_parts <= 64, "key_parts must be in [1, 64]");
    COME_REQUIRE(lse_parts_dev != nullptr || q_rows == 0, "come_attn_cross_fwd_parts needs the log-sum-exp output");
    const int max_len = (int)(kv_rows < (1ll << 31) ? kv_rows : 0);
    const int64_t row_stride = (int64_t)num_heads * head_dim;  // every share is a contiguous [q_rows, num_heads, head_dim] block
    return attn_dispatch(q_dev, k_dev, v_dev, dtype, kv_rows, 0, q_rows, num_heads, head_dim, q_row_stride, k_row_stride,
                         v_row_stride, bias_dev, nullptr, 1, max_len, nullptr, softmax_scale, out_parts_dev, row_stride,
                         lse_parts_dev, backend, stream, true, key_parts, q_rows * row_stride);
}

extern "C" int come_attn_combine_parts(const void *out_parts_dev, const float *lse_parts_dev, int key_parts, int dtype,
                                       int64_t rows, int num_heads, int head_dim, void *out_dev, float *lse_out_dev,
                                       void *stream) {
    COME_REQUIRE(dtype == COME_F16 || dtype == COME_BF16, "come_attn_combine_parts: dtype must be COME_F16 or COME_BF16");
    COME_REQUIRE(key_parts >= 1 && rows >= 0 && num_heads > 0 && head_dim > 0 && head_dim % 8 == 0, "come_attn_combine_parts: bad shape");
    if (rows == 0) return COME_OK;
    COME_REQUIRE(out_parts_dev && lse_parts_dev && out_dev, "come_attn_combine_parts: NULL pointer");
    COME_REQUIRE(((uintptr_t)out_parts_dev & 15) == 0 && ((uintptr_t)out_dev & 15) == 0, "come_attn_combine_parts: outputs must be 16-byte aligned");
    const int64_t n = rows * num_heads * (head_dim / 8);
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t part_o = rows * num_heads * head_dim;
    if (dtype == COME_F16)
        attn_combine_parts_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half *)out_parts_dev, lse_parts_dev, key_parts, part_o,
                                                                          rows, num_heads, head_dim, (__half *)out_dev, lse_out_dev);
    else
        attn_combine_parts_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16 *)out_parts_dev, lse_parts_dev,
                                                                                 key_parts, part_o, rows, num_heads, head_dim,
                                                                                 (__nv_bfloat16 *)out_dev, lse_out_dev);
    return check_launch("come_attn_combine_parts");
}

extern "C" int come_attn_combine(const void *out_a_dev, const float *lse_a_dev, const void *out_b_dev, const float *lse_b_dev,
                                 int dtype, int64_t rows, int num_heads, int head_dim, void *out_dev, float *lse_out_dev,
                                 void *stream) {
    COME_REQUIRE(dtype == COME_F16 || dtype == COME_BF16, "come_attn_combine: dtype must be COME_F16 or COME_BF16");
    COME_REQUIRE(rows >= 0 && num_heads > 0 && head_dim > 0 && head_dim % 8 == 0, "come_attn_combine: bad shape");
    if (rows == 0) return COME_OK;
    COME_REQUIRE(out_a_dev && out_b_dev && lse_a_dev && lse_b_dev && out_dev, "come_attn_combine: NULL pointer");
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    COME_REQUIRE(al16(out_a_dev) && al16(out_b_dev) && al16(out_dev), "come_attn_combine: outputs must be 16-byte aligned");
    const int64_t n = rows * num_heads * (head_dim / 8);
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == COME_F16)
        attn_combine_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half *)out_a_dev, lse_a_dev, (const __half *)out_b_dev,
                                                                    lse_b_dev, rows, num_heads, head_dim, (__half *)out_dev, lse_out_dev);
    else
        attn_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16 *)out_a_dev, lse_a_dev,
                                                                           (const __nv_bfloat16 *)out_b_dev, lse_b_dev, rows,
                                                                           num_heads, head_dim, (__nv_bfloat16 *)out_dev, lse_out_dev);
    return check_launch("come_attn_combine");
}

extern "C" int come_attn_set_cta_limit(int max_ctas) {
    COME_REQUIRE(max_ctas >= 0, "come_attn_set_cta_limit: max_ctas must be >= 0");
    attn_sm100_set_cta_limit(max_ctas);
    return COME_OK;
}
