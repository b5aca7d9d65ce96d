// Token merge / unmerge for sm_100a: index plan, packed-row gather with window means, row gather back.
//
// All three data kernels are HBM-bandwidth bound.  They move 16-byte vectors, keep a full window's loads
// in flight per thread before the first add, and run as persistent grid-stride loops sized to the SM count.
#include <type_traits>

#include "come_internal.cuh"

#include <cstdlib>
#include <mutex>

namespace come {

// ---- common host state -------------------------------------------------------------------------------------
static thread_local char t_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

static __device__ unsigned int g_status_word = 0;

unsigned int *status_word_dev() {
    static unsigned int *cached[64];  // looked up once per device (keeps later calls legal inside a stream capture)
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice failed or device index out of range");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        unsigned int *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_status_word);
        if (e != cudaSuccess) {
            set_error("cudaGetSymbolAddress(status word) failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev] = p;
    }
    return cached[dev];
}

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int make_layout(const come_layout_t *in, FrameLayout *out) {
    COME_REQUIRE(in != nullptr, "layout is NULL");
    COME_REQUIRE(in->start_index >= 0, "start_index must be >= 0, got %d", in->start_index);
    FrameLayout L{};
    L.start = in->start_index;
    if (in->grid_h == 0) {
        COME_REQUIRE(in->group_w > 0, "group_size must be > 0, got %d", in->group_w);
        COME_REQUIRE(in->n_groups >= 0, "n_groups must be >= 0, got %d", in->n_groups);
        L.H = 0;
        L.W = 0;
        L.gh = 1;
        L.gw = in->group_w;
        L.G = in->group_w;
        L.M = in->n_groups;
        L.Wm = in->n_groups;
        L.prefix = in->start_index;
        L.N = (int)((int64_t)L.start + (int64_t)L.M * L.G);
        COME_REQUIRE((int64_t)L.start + (int64_t)L.M * L.G < (1ll << 31), "frame too long");
    } else {
        COME_REQUIRE(in->grid_h > 0 && in->grid_w > 0, "grid must be positive, got (%d, %d)", in->grid_h, in->grid_w);
        COME_REQUIRE(in->group_h > 0 && in->group_w > 0, "group_h and group_w must be > 0, got (%d, %d)",
                     in->group_h, in->group_w);
        COME_REQUIRE((int64_t)in->grid_h * in->grid_w + in->start_index < (1ll << 31), "frame too long");
        L.H = in->grid_h;
        L.W = in->grid_w;
        L.gh = in->group_h;
        L.gw = in->group_w;
        L.G = in->group_h * in->group_w;
        L.Wm = L.W / L.gw;
        L.Hc = (L.H / L.gh) * L.gh;
        L.Wc = L.Wm * L.gw;
        L.edge_cols = L.W - L.Wc;
        L.M = (L.H / L.gh) * L.Wm;
        L.N = L.start + L.H * L.W;
        L.prefix = L.N - L.M * L.G;
    }
    *out = L;
    return COME_OK;
}

// ---- index plan ------------------------------------------------------------------------------------------------
// Pass 1: one warp per frame counts the merged windows of its row and records the packed frame length.
__global__ void plan_count_kernel(const uint8_t *__restrict__ mask, int frames, int M, int G, int prefix,
                                  int *__restrict__ frame_len) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= frames) return;
    const uint8_t *row = mask + (size_t)warp * M;
    int k = 0;
    for (int m = lane; m < M; m += 32) k += row[m] != 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
    if (lane == 0) frame_len[warp] = prefix + (M - k) * G + k;
}

// Pass 2: one CTA per frame.  Sums the lengths of the preceding frames (its packed base row), scans its own
// row of the mask, and writes group_prefix, offsets, rev_id and weight.
constexpr int kPlanThreads = 256;

__global__ void __launch_bounds__(kPlanThreads)
plan_write_kernel(const uint8_t *__restrict__ mask, const int *__restrict__ frame_len, int frames, FrameLayout L,
                  int *__restrict__ group_prefix, int *__restrict__ offsets, int64_t *__restrict__ rev,
                  float *__restrict__ weight, int *__restrict__ seg_max) {
    __shared__ int s_warp[kPlanThreads / 32];
    __shared__ int s_base, s_carry;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;

    // packed base row of this frame = sum of the lengths of frames [0, b)
    int part = 0, mx = 0;
    const int upto = (b == 0) ? frames : b;  // CTA 0 also produces the grand total and the longest frame
    for (int i = tid; i < upto; i += kPlanThreads) {
        int len = frame_len[i];
        part += len;
        mx = max(mx, len);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        part += __shfl_xor_sync(0xffffffffu, part, o);
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ int s_max[kPlanThreads / 32];
    if (lane == 0) {
        s_warp[wid] = part;
        s_max[wid] = mx;
    }
    __syncthreads();
    if (tid == 0) {
        int tot = 0, m2 = 0;
        for (int w = 0; w < kPlanThreads / 32; ++w) {
            tot += s_warp[w];
            m2 = max(m2, s_max[w]);
        }
        if (b == 0) {
            offsets[frames] = tot;
            offsets[0] = 0;
            if (seg_max) *seg_max = m2;
            s_base = 0;
        } else {
            offsets[b] = tot;
            s_base = tot;
        }
        s_carry = 0;
    }
    __syncthreads();
    const int base = s_base;
    const int64_t tok0 = (int64_t)b * L.N;

    // never-merged prefix rows
    for (int s = tid; s < L.prefix; s += kPlanThreads) {
        rev[tok0 + L.src_token(s)] = base + s;
        weight[base + s] = 1.0f;
    }

    // exclusive scan of (mask ? 1 : G) over the M groups, tile by tile
    const uint8_t *row = mask + (size_t)b * L.M;
    for (int t0 = 0; t0 < L.M; t0 += kPlanThreads) {
        const int m = t0 + tid;
        const bool valid = m < L.M;
        const bool merged = valid && row[m] != 0;
        const int len = valid ? (merged ? 1 : L.G) : 0;
        int incl = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        __syncthreads();  // s_warp / s_carry of the previous tile fully consumed
        if (lane == 31) s_warp[wid] = incl;
        __syncthreads();
        int warp_off = 0;
        for (int w = 0; w < wid; ++w) warp_off += s_warp[w];
        const int excl = s_carry + warp_off + incl - len;
        if (valid) {
            group_prefix[(size_t)b * L.M + m] = excl;
            const int dst = base + L.prefix + excl;
            const int r0 = L.prefix + m * L.G;
            if (merged) {
                weight[dst] = (float)L.G;
                for (int g = 0; g < L.G; ++g) rev[tok0 + L.src_token(r0 + g)] = dst;
            } else {
                for (int g = 0; g < L.G; ++g) {
                    weight[dst + g] = 1.0f;
                    rev[tok0 + L.src_token(r0 + g)] = dst + g;
                }
            }
        }
        __syncthreads();
        if (tid == kPlanThreads - 1) s_carry = excl + len;  // total of this tile carried to the next
    }
}

// ---- merge data movement ----------------------------------------------------------------------------------------
// One work unit = one window (G source rows) or one chunk of up to G prefix rows.  A CTA walks units with a
// grid stride; inside a unit a thread owns 16-byte column vectors.  VEC = elements per vector (1 = scalar path
// for rows that are not 16-byte multiples).
constexpr int kMergeThreads = 256;
constexpr int kMaxInFlight = 9;   // rows whose loads are issued before the first add / store

template <typename T, int VEC> struct VecIO;
template <> struct VecIO<float, 4> {
    using V = float4;
    static __device__ __forceinline__ void unpack(const V &v, float (&f)[4]) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
    static __device__ __forceinline__ V pack(const float (&f)[4]) { return make_float4(f[0], f[1], f[2], f[3]); }
};
template <typename T> struct VecIO<T, 8> {  // __half / __nv_bfloat16
    using V = uint4;
    static __device__ __forceinline__ void unpack(const V &v, float (&f)[8]) {
        const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = Elem<T>::to_f32(e[i]);
    }
    static __device__ __forceinline__ V pack(const float (&f)[8]) {
        V v;
        T *e = reinterpret_cast<T *>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = Elem<T>::from_f32(f[i]);
        return v;
    }
};
template <typename T> struct VecIO<T, 1> {
    using V = T;
    static __device__ __forceinline__ void unpack(const V &v, float (&f)[1]) { f[0] = Elem<T>::to_f32(v); }
    static __device__ __forceinline__ V pack(const float (&f)[1]) { return Elem<T>::from_f32(f[0]); }
};

template <typename V> __device__ __forceinline__ V ld_stream(const V *p) { return __ldcs(p); }
template <> __device__ __forceinline__ __half ld_stream<__half>(const __half *p) { return *p; }
template <> __device__ __forceinline__ __nv_bfloat16 ld_stream<__nv_bfloat16>(const __nv_bfloat16 *p) { return *p; }
template <typename V> __device__ __forceinline__ void st_stream(V *p, const V &v) { __stcs(p, v); }
template <> __device__ __forceinline__ void st_stream<__half>(__half *p, const __half &v) { *p = v; }
template <> __device__ __forceinline__ void st_stream<__nv_bfloat16>(__nv_bfloat16 *p, const __nv_bfloat16 &v) { *p = v; }

// INFLIGHT = rows whose loads are issued before the first add / store, MINB = CTAs per SM the registers are held to:
// (9, 2) streams best on launches of several waves; (5, 4) doubles the resident CTAs, which is what a launch of one or
// two waves (a single 8-frame scene) needs to hide its three dependent memory round trips per unit.
template <typename T, int VEC, int INFLIGHT, int MINB>
__global__ void __launch_bounds__(kMergeThreads, MINB)
merge_kernel(const T *__restrict__ tokens, const uint8_t *__restrict__ mask, const int *__restrict__ group_prefix,
             const int *__restrict__ offsets, FrameLayout L, int frames, int64_t C, int groups, T *__restrict__ out) {
    using IO = VecIO<T, VEC>;
    using V = typename IO::V;
    extern __shared__ int s_src_all[];  // source token of every row of the current unit, per thread group (groups x G)
    const int G = L.G;
    // Rows narrower than the CTA (e.g. 1024 x 16-bit = 128 vectors): the host splits the CTA into `groups` thread
    // groups of `tpg` threads (whole warps), each moving its own unit, so that no thread idles.
    const int tpg = kMergeThreads / groups;
    const int grp = threadIdx.x / tpg, tig = threadIdx.x - grp * tpg;
    int *s_src = s_src_all + grp * G;
    const int prefix_units = (L.prefix + G - 1) / G;
    const int units_per_frame = prefix_units + L.M;
    const int n_units = frames * units_per_frame;  // fits: the host checks frames * tokens_per_frame < 2^31
    const int64_t Cv = C / VEC;
    const float fG = (float)G;

    for (int u0 = blockIdx.x * groups; u0 < n_units; u0 += gridDim.x * groups) {
        const int u = u0 + grp;
        const bool active = u < n_units;  // the last round may leave some groups without a unit
        const int b = active ? u / units_per_frame : 0;
        const int unit = active ? u - b * units_per_frame : 0;
        const int base = offsets[b];
        int r0, rows, dst;
        bool merged = false;
        if (!active) {
            r0 = 0;
            rows = 0;
            dst = 0;
        } else if (unit < prefix_units) {
            r0 = unit * G;
            rows = min(G, L.prefix - r0);
            dst = base + r0;
        } else {
            const int m = unit - prefix_units;
            r0 = L.prefix + m * G;
            rows = G;
            dst = base + L.prefix + group_prefix[(size_t)b * L.M + m];
            merged = mask[(size_t)b * L.M + m] != 0;
        }
        __syncthreads();  // previous unit's s_src no longer read
        for (int g = tig; g < rows; g += tpg) s_src[g] = L.src_token(r0 + g);
        __syncthreads();
        const V *src_base = reinterpret_cast<const V *>(tokens) + (int64_t)b * L.N * Cv;
        V *dst_base = reinterpret_cast<V *>(out) + (int64_t)dst * Cv;

        for (int64_t v = tig; v < Cv && active; v += tpg) {
            if (merged) {
                float acc[VEC];
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
                for (int g0 = 0; g0 < rows; g0 += INFLIGHT) {
                    V buf[INFLIGHT];
#pragma unroll
                    for (int i = 0; i < INFLIGHT; ++i)
                        if (g0 + i < rows) buf[i] = ld_stream(src_base + (int64_t)s_src[g0 + i] * Cv + v);
#pragma unroll
                    for (int i = 0; i < INFLIGHT; ++i)
                        if (g0 + i < rows) {
                            float f[VEC];
                            IO::unpack(buf[i], f);
#pragma unroll
                            for (int j = 0; j < VEC; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
                        }
                }
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[j] = __fdiv_rn(acc[j], fG);
                st_stream(dst_base + v, IO::pack(acc));
            } else {
                for (int g0 = 0; g0 < rows; g0 += INFLIGHT) {
                    V buf[INFLIGHT];
#pragma unroll
                    for (int i = 0; i < INFLIGHT; ++i)
                        if (g0 + i < rows) buf[i] = ld_stream(src_base + (int64_t)s_src[g0 + i] * Cv + v);
#pragma unroll
                    for (int i = 0; i < INFLIGHT; ++i)
                        if (g0 + i < rows) st_stream(dst_base + (int64_t)(g0 + i) * Cv + v, buf[i]);
                }
            }
        }
    }
}


// ---- merge through a shared-memory ring fed by bulk copies -----------------------------------------------------------
// For rows that are multiples of 16 bytes and units (G rows) that fit the ring: one persistent CTA per SM; a producer lane
// copies every unit's source rows global -> shared with plain bulk copies (cp.async.bulk, no tensor map: a 3 x 3 window
// of a row-major grid is three runs of three consecutive tokens, a 1-D group is one run) into a ring several units deep,
// so that ~150 KB per SM are in flight all the time instead of two CTAs alternating load / add / store phases.  Kept
// windows and prefix rows leave the ring by a bulk copy shared -> global issued by a second lane (their packed rows are
// consecutive); merged windows are summed from shared memory by four consumer warps in the fixed left-to-right order of
// merge_kernel (float32 sum, IEEE division, one rounding) and stored from registers.  Every wait is bounded.
constexpr int kBulkThreads = 256;       // warps 0-1: producers, warps 2-3: bulk stores (one lane each), warps 4-7: consumers
constexpr int kBulkLanes = 2;           // producers and store lanes work on alternate units: unit k belongs to lane k % 2
constexpr int kBulkConsumers = 128;
constexpr int kBulkMaxStages = 8;       // a multiple of kBulkLanes, see launch_merge
constexpr long long kBulkWaitTicks = 1ll << 29;
constexpr unsigned kErrMergeBulk = 1u << 17;  // device status bit of a wait that ran out in merge_bulk_kernel

__device__ __forceinline__ uint32_t cvta_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool bulk_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(cvta_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bulk_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag, unsigned int *status) {
    if (bulk_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (bulk_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > kBulkWaitTicks) {
            *abort_flag = 1;
            atomicOr(status, kErrMergeBulk);
            return false;
        }
    }
}

// What the producer publishes about a unit, in shared memory beside its stage: the other roles read it after the stage's
// "full" barrier instead of decoding the unit from global memory themselves (three dependent loads per unit).
struct BulkUnit {
    int dst;      // first packed row
    int rows;     // source rows in the stage
    int merged;   // window mean (consumers) or plain copy (store lane)
    int pad;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(kBulkThreads, 1)
merge_bulk_kernel(const T *__restrict__ tokens, const uint8_t *__restrict__ mask, const int *__restrict__ group_prefix,
                  const int *__restrict__ offsets, FrameLayout L, int frames, int64_t C, int stages, T *__restrict__ out,
                  unsigned int *__restrict__ status) {
    using IO = VecIO<T, VEC>;
    using V = typename IO::V;
    extern __shared__ __align__(128) uint8_t bulk_smem[];
    const int G = L.G;
    const uint32_t row_bytes = (uint32_t)(C * sizeof(T));
    const uint32_t stage_bytes = (uint32_t)G * row_bytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(bulk_smem + (size_t)stages * stage_bytes);
    uint64_t *empty = full + stages;
    BulkUnit *desc = reinterpret_cast<BulkUnit *>(empty + stages);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(desc + stages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < stages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(cvta_smem(&full[i])), "r"(1));
            // every unit is released by all consumer threads and by the store lane, whichever of them used it
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(cvta_smem(&empty[i])), "r"(kBulkConsumers + 1));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int prefix_units = (L.prefix + G - 1) / G;
    const int units_per_frame = prefix_units + L.M;
    const int n_units = frames * units_per_frame;
    const int my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp < kBulkLanes) {
        // ===== producers: the 32 lanes decode 32 units at a time (their global loads overlap), then the units' bulk loads are
        // issued in order; producer p owns the units k = p, p + 2, ... of this CTA =====
        const int p = warp;
        const int mine = my_units > p ? (my_units - p + kBulkLanes - 1) / kBulkLanes : 0;
        bool ok = true;
        for (int j0 = 0; j0 < mine && ok; j0 += 32) {
            const int jj = j0 + lane;
            int b = 0, r0 = 0, rows = 0, dst = 0, merged = 0;
            if (jj < mine) {
                const int u = blockIdx.x + (p + kBulkLanes * jj) * gridDim.x;
                b = u / units_per_frame;
                const int unit = u - b * units_per_frame;
                const int base = offsets[b];
                if (unit < prefix_units) {
                    r0 = unit * G;
                    rows = min(G, L.prefix - r0);
                    dst = base + r0;
                } else {
                    const int m = unit - prefix_units;
                    r0 = L.prefix + m * G;
                    rows = G;
                    dst = base + L.prefix + group_prefix[(size_t)b * L.M + m];
                    merged = mask[(size_t)b * L.M + m] != 0;
                }
            }
            const int n_here = min(32, mine - j0);
            for (int i = 0; i < n_here && ok; ++i) {
                const int k = p + kBulkLanes * (j0 + i), stage = k % stages;
                const int ub = __shfl_sync(0xffffffffu, b, i), ur0 = __shfl_sync(0xffffffffu, r0, i);
                const int urows = __shfl_sync(0xffffffffu, rows, i), udst = __shfl_sync(0xffffffffu, dst, i);
                const int umerged = __shfl_sync(0xffffffffu, merged, i);
                // Source token of every row of the unit, one row per lane (the index arithmetic divides several times), and
                // the rows that start a run of consecutive tokens: a run travels as one copy, issued by the lane of its
                // first row, so the copies of a unit are issued side by side.
                const int tok = lane < urows ? L.src_token(ur0 + lane) : -1;
                const int prev = __shfl_up_sync(0xffffffffu, tok, 1);
                const bool is_start = lane < urows && (lane == 0 || tok != prev + 1);
                const unsigned starts = __ballot_sync(0xffffffffu, is_start);
                const unsigned above = lane < 31 ? (starts & ~((2u << lane) - 1u)) : 0u;
                const int run_end = above != 0 ? __ffs(above) - 1 : urows;
                if (lane == 0) {
                    if (k >= stages) ok = bulk_wait(&empty[stage], ((k / stages) - 1) & 1, abort_flag, status);
                    if (ok) {
                        desc[stage] = BulkUnit{udst, urows, umerged, 0};  // ordered before the loads' completion by the arrive below
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(cvta_smem(&full[stage])), "r"((uint32_t)urows * row_bytes) : "memory");
                    }
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;  // also orders the expect_tx in front of the copies below
                if (ok && is_start) {
                    const uint8_t *frame = reinterpret_cast<const uint8_t *>(tokens) + (size_t)ub * L.N * row_bytes;
                    uint8_t *dst_s = bulk_smem + (size_t)stage * stage_bytes;
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(cvta_smem(dst_s + (size_t)lane * row_bytes)), "l"(frame + (size_t)tok * row_bytes),
                                   "r"((uint32_t)(run_end - lane) * row_bytes), "r"(cvta_smem(&full[stage])) : "memory");
                }
            }
        }
    } else if (warp < 2 * kBulkLanes) {
        // ===== store lanes: units that are copied unchanged leave the ring by one bulk store; store lane q owns the units
        // k = q, q + 2, ... =====
        if (lane == 0) {
            int pending_stage = -1;
            for (int k = warp - kBulkLanes; k < my_units; k += kBulkLanes) {
                const int stage = k % stages;
                // Every role waits for every unit's data before it releases the unit, also when the unit is not its own: a
                // role that released units it does not use without waiting would run ahead, arrive for the stage's NEXT
                // unit while the current one is still being read, and complete the phase early.
                if (!bulk_wait(&full[stage], (k / stages) & 1, abort_flag, status)) break;
                const BulkUnit d = desc[stage];
                if (d.merged) {  // the consumers' unit: nothing to store
                    if (pending_stage >= 0) {
                        // no store follows at once: hand the last store's stage back now (the producer may need it soon)
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cvta_smem(&empty[pending_stage])) : "memory");
                        pending_stage = -1;
                    }
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cvta_smem(&empty[stage])) : "memory");
                    continue;
                }
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(reinterpret_cast<uint8_t *>(out) + (size_t)d.dst * row_bytes),
                               "r"(cvta_smem(bulk_smem + (size_t)stage * stage_bytes)), "r"((uint32_t)d.rows * row_bytes) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                if (pending_stage >= 0) {  // the store before this one has read its stage: hand it back
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cvta_smem(&empty[pending_stage])) : "memory");
                }
                pending_stage = stage;
            }
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            if (pending_stage >= 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cvta_smem(&empty[pending_stage])) : "memory");
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores complete before the CTA's shared memory goes away
        }
    } else {
        // ===== consumers: window means =====
        const int tid = threadIdx.x - 2 * kBulkLanes * 32;
        const int64_t Cv = C / VEC;
        const float fG = (float)G;
        for (int k = 0; k < my_units; ++k) {
            const int stage = k % stages;
            if (!bulk_wait(&full[stage], (k / stages) & 1, abort_flag, status)) break;  // see the store lane
            const BulkUnit d = desc[stage];
            if (d.merged) {
                const V *src = reinterpret_cast<const V *>(bulk_smem + (size_t)stage * stage_bytes);
                V *dst_row = reinterpret_cast<V *>(out) + (int64_t)d.dst * Cv;
                for (int64_t v = tid; v < Cv; v += kBulkConsumers) {
                    float acc[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
                    for (int g = 0; g < d.rows; ++g) {
                        float f[VEC];
                        IO::unpack(src[(int64_t)g * Cv + v], f);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
                    }
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc[j] = __fdiv_rn(acc[j], fG);
                    st_stream(dst_row + v, IO::pack(acc));
                }
            }
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cvta_smem(&empty[stage])) : "memory");
        }
    }
}

// The bulk-ring kernel can be switched off (COME_MERGE_BULK=0 in the environment, read once) to compare the two merge
// kernels; they produce the same bits.
// COME_MERGE_LN_ROWS=0 in the environment keeps the thread-group LayerNorm + merge kernel for every row width (A/B runs).
static bool ln_rows_disabled() {
    static const bool off = [] {
        const char *e = getenv("COME_MERGE_LN_ROWS");
        return e != nullptr && e[0] == '0';
    }();
    return off;
}
static bool bulk_disabled() {
    static const bool off = [] {
        const char *v = getenv("COME_MERGE_BULK");
        return v != nullptr && v[0] == '0';
    }();
    return off;
}

// Shared-memory opt-in of the bulk-ring kernel: raised per device and instantiation when a launch needs more than before.
template <typename T, int VEC> static int ensure_bulk_smem(size_t smem) {
    static std::mutex mu;
    static size_t have[64];
    int dev = 0;
    COME_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("come_merge: device ordinal %d is out of the supported range", dev);
        return COME_ERR_ARG;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (have[dev] >= smem) return COME_OK;
    COME_CUDA(cudaFuncSetAttribute(merge_bulk_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024)));
    have[dev] = 220 * 1024;
    return COME_OK;
}

// ---- merge fused with the LayerNorm in front of it ---------------------------------------------------------------
// out = merge(LayerNorm(tokens)): every source row is normalised over its C channels (float32 statistics and affine map,
// result rounded to T like the module's output tensor), then merged windows average their G normalised rows.  One
// thread group of `tpg` threads (a power of two >= the vectors per row) owns a unit; a thread holds its 16-byte vector
// of every row of the unit in registers as float32 pairs, so the tokens are read once.
//
// Summation order of a row's statistics (fixed, so that the CPU oracle can follow it bit for bit): inside a thread the
// even and the odd channels of its vector are summed left to right as two chains (packed two-lane adds) and the chains
// added; the threads' partial sums go through shared memory, where one warp per row adds, for every lane position, the
// partials of the group's warps left to right and then runs a butterfly over the 32 lanes (neighbours first).  The
// squares are accumulated with fused multiply-adds.  The same warp turns the totals into mean and 1/sqrt(var + eps).
constexpr int kRowWarps = 8;   // warps per CTA of the warp-per-row kernels
constexpr int kLnMaxRows = 9;  // rows per unit the fused kernel keeps in registers (3 x 3 windows)

__device__ __forceinline__ void group_barrier(int groups, int grp, int tpg) {
    if (groups == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(tpg) : "memory");
}

template <typename T, int VEC> struct PairIO;  // 16-byte vector <-> VEC/2 float32 pairs
template <> struct PairIO<float, 4> {
    static __device__ __forceinline__ void unpack(const float4 &v, f32x2_t (&p)[2]) {
        p[0] = pack_f32x2(v.x, v.y);
        p[1] = pack_f32x2(v.z, v.w);
    }
    static __device__ __forceinline__ float4 pack(const f32x2_t (&p)[2]) {
        float4 v;
        unpack_f32x2(p[0], v.x, v.y);
        unpack_f32x2(p[1], v.z, v.w);
        return v;
    }
    static __device__ __forceinline__ f32x2_t round_pair(f32x2_t p) { return p; }
};
// 16-bit pairs <-> float32 pairs on 32-bit words (no address-taken arrays: everything stays in registers).
__device__ __forceinline__ float2 word_to_f32(uint32_t w, __half) { return __half22float2(*reinterpret_cast<const __half2 *>(&w)); }
__device__ __forceinline__ float2 word_to_f32(uint32_t w, __nv_bfloat16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));  // a bfloat16 is the top half of a float32
}
__device__ __forceinline__ uint32_t f32_to_word(float lo, float hi, __half) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t f32_to_word(float lo, float hi, __nv_bfloat16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
template <typename T> struct PairIO16 {
    static __device__ __forceinline__ void unpack(const uint4 &v, f32x2_t (&p)[4]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = word_to_f32(w[j], T());
            p[j] = pack_f32x2(f.x, f.y);
        }
    }
    static __device__ __forceinline__ uint4 pack(const f32x2_t (&p)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float lo, hi;
            unpack_f32x2(p[j], lo, hi);
            w[j] = f32_to_word(lo, hi, T());
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ f32x2_t round_pair(f32x2_t p) {
        float lo, hi;
        unpack_f32x2(p, lo, hi);
        const float2 f = word_to_f32(f32_to_word(lo, hi, T()), T());
        return pack_f32x2(f.x, f.y);
    }
};
template <> struct PairIO<__half, 8> : PairIO16<__half> {};
template <> struct PairIO<__nv_bfloat16, 8> : PairIO16<__nv_bfloat16> {};

// TPG > 0: the thread-group size is a compile-time constant equal to the vectors per row (every thread has a column,
// shared-memory offsets are constants, the warp loops unroll); TPG == 0: any row width, sizes at run time.
template <typename T, int VEC, int TPG>
__global__ void __launch_bounds__(kMergeThreads, 2)
merge_layernorm_kernel(const T *__restrict__ tokens, const uint8_t *__restrict__ mask, const int *__restrict__ group_prefix,
                       const int *__restrict__ offsets, FrameLayout L, int frames, int Cv, int groups,
                       const T *__restrict__ gamma, const T *__restrict__ beta, float eps, T *__restrict__ out) {
    using IO = VecIO<T, VEC>;
    using PIO = PairIO<T, VEC>;
    using V = typename IO::V;
    constexpr int NP = VEC / 2;  // float32 pairs per thread and row
    extern __shared__ int s_ln_raw[];
    const int G = L.G;
    const int tpg = TPG > 0 ? TPG : kMergeThreads / groups, warps_pg = tpg / 32;
    if constexpr (TPG > 0) groups = kMergeThreads / TPG;
    const int grp = threadIdx.x / tpg, tig = threadIdx.x - grp * tpg;
    const int wig = tig >> 5, lane = tig & 31;
    // shared memory: [groups][G] source tokens | [groups][kLnMaxRows][tpg] partial sums | [groups][kLnMaxRows] row statistic
    int *s_src = s_ln_raw + grp * G;
    float *s_part = reinterpret_cast<float *>(s_ln_raw + groups * G) + grp * (kLnMaxRows * tpg);
    float *s_stat = reinterpret_cast<float *>(s_ln_raw + groups * G) + groups * (kLnMaxRows * tpg) + grp * kLnMaxRows;
    const int prefix_units = (L.prefix + G - 1) / G;
    const int units_per_frame = prefix_units + L.M;
    const int n_units = frames * units_per_frame;
    const bool has_col = TPG > 0 || tig < Cv;  // a run-time group may be wider than a row (rows of 96, 192, ... vectors)
    const float fC = (float)(Cv * VEC), fG = (float)G;
    V g_raw = V(), b_raw = V();  // this thread's gamma / beta, kept packed (unpacked where used: registers are tight)
    if (has_col) {
        g_raw = reinterpret_cast<const V *>(gamma)[tig];
        b_raw = reinterpret_cast<const V *>(beta)[tig];
    }

    // Row totals of one partial sum per thread, for all rows of the unit at once; `finish` turns a row's total into the
    // statistic every thread then reads back (mean after the first pass, 1/sqrt(var + eps) after the second).
    auto row_statistics = [&](float (&part)[kLnMaxRows], const int rows, auto finish) {
        group_barrier(groups, grp, tpg);  // the previous use of s_part / s_stat is over
#pragma unroll
        for (int r = 0; r < kLnMaxRows; ++r)
            if (r < rows) s_part[r * tpg + tig] = part[r];
        group_barrier(groups, grp, tpg);
        for (int r = wig; r < rows; r += warps_pg) {
            float t = s_part[r * tpg + lane];
            for (int w = 1; w < warps_pg; ++w) t = __fadd_rn(t, s_part[r * tpg + w * 32 + lane]);
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, m));
            if (lane == 0) s_stat[r] = finish(t);
        }
        group_barrier(groups, grp, tpg);
#pragma unroll
        for (int r = 0; r < kLnMaxRows; ++r) part[r] = (r < rows) ? s_stat[r] : 0.0f;
    };

    for (int u0 = blockIdx.x * groups; u0 < n_units; u0 += gridDim.x * groups) {
        const int u = u0 + grp;
        const bool active = u < n_units;  // the last round may leave some groups without a unit (they still meet the barriers)
        const int bfr = active ? u / units_per_frame : 0;
        const int unit = active ? u - bfr * units_per_frame : 0;
        const int base = offsets[bfr];
        int r0 = 0, rows = 0, dst = 0;
        bool merged = false;
        if (active) {
            if (unit < prefix_units) {
                r0 = unit * G;
                rows = min(G, L.prefix - r0);
                dst = base + r0;
            } else {
                const int m = unit - prefix_units;
                r0 = L.prefix + m * G;
                rows = G;
                dst = base + L.prefix + group_prefix[(size_t)bfr * L.M + m];
                merged = mask[(size_t)bfr * L.M + m] != 0;
            }
        }
        group_barrier(groups, grp, tpg);  // previous unit's s_src no longer read
        for (int r = tig; r < rows; r += tpg) s_src[r] = L.src_token(r0 + r);
        group_barrier(groups, grp, tpg);
        // A unit of kLnMaxRows rows (every 3 x 3 window) takes the copy of the body below in which the row count is a
        // constant: no per-row predicates are left.
        const bool full = (rows == kLnMaxRows);
        auto process = [&](auto full_tag) {
        constexpr bool FULL = decltype(full_tag)::value;
        const int n_rows = FULL ? kLnMaxRows : rows;
        const V *src_base = reinterpret_cast<const V *>(tokens) + (int64_t)bfr * L.N * Cv;

        V raw[kLnMaxRows];
#pragma unroll
        for (int r = 0; r < kLnMaxRows; ++r)
            if ((FULL || r < n_rows) && has_col) raw[r] = ld_stream(src_base + (int64_t)s_src[r] * Cv + tig);
        f32x2_t x[kLnMaxRows][NP];
        float stat[kLnMaxRows];
#pragma unroll
        for (int r = 0; r < kLnMaxRows; ++r) {
            stat[r] = 0.0f;
#pragma unroll
            for (int j = 0; j < NP; ++j) x[r][j] = 0ull;
            if ((FULL || r < n_rows) && has_col) {
                PIO::unpack(raw[r], x[r]);
                f32x2_t acc = x[r][0];
#pragma unroll
                for (int j = 1; j < NP; ++j) acc = add_f32x2(acc, x[r][j]);
                float even, odd;
                unpack_f32x2(acc, even, odd);
                stat[r] = __fadd_rn(even, odd);
            }
        }
        row_statistics(stat, n_rows, [&](float total) { return __fdiv_rn(total, fC); });
#pragma unroll
        for (int r = 0; r < kLnMaxRows; ++r) {
            const f32x2_t neg_mean = pack_f32x2(-stat[r], -stat[r]);
            stat[r] = 0.0f;
            if ((FULL || r < n_rows) && has_col) {
#pragma unroll
                for (int j = 0; j < NP; ++j) x[r][j] = add_f32x2(x[r][j], neg_mean);  // x - mean
                f32x2_t acc = mul_f32x2(x[r][0], x[r][0]);
#pragma unroll
                for (int j = 1; j < NP; ++j) acc = fma_f32x2(x[r][j], x[r][j], acc);  // explicit: never a separate mul + add
                float even, odd;
                unpack_f32x2(acc, even, odd);
                stat[r] = __fadd_rn(even, odd);
            }
        }
        row_statistics(stat, n_rows, [&](float total) { return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, fC), eps))); });
        if (has_col) {
            f32x2_t acc[NP], g2[NP], b2[NP];
            PIO::unpack(g_raw, g2);
            PIO::unpack(b_raw, b2);
#pragma unroll
            for (int j = 0; j < NP; ++j) acc[j] = 0ull;
            V *dst_base = reinterpret_cast<V *>(out) + (int64_t)dst * Cv + tig;
#pragma unroll
            for (int r = 0; r < kLnMaxRows; ++r) {
                if ((FULL || r < n_rows)) {
                    const f32x2_t rstd2 = pack_f32x2(stat[r], stat[r]);
#pragma unroll
                    for (int j = 0; j < NP; ++j) x[r][j] = fma_f32x2(g2[j], mul_f32x2(rstd2, x[r][j]), b2[j]);
                    if (merged) {
                        // the normalised tensor lives in T: its rounded values are what the window mean sums
#pragma unroll
                        for (int j = 0; j < NP; ++j) acc[j] = add_f32x2(acc[j], PIO::round_pair(x[r][j]));
                    } else {
                        st_stream(dst_base + (int64_t)r * Cv, PIO::pack(x[r]));
                    }
                }
            }
            if (merged) {
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    float lo, hi;
                    unpack_f32x2(acc[j], lo, hi);
                    acc[j] = pack_f32x2(__fdiv_rn(lo, fG), __fdiv_rn(hi, fG));
                }
                st_stream(dst_base, PIO::pack(acc));
            }
        }
        };  // process
        if (full) process(std::true_type{});
        else process(std::false_type{});
    }
}

// The same operation with one WARP per unit: lane l holds the 16-byte vectors l, l + 32, ... of a row (NV of them), the
// unit's rows are taken one after the other (the next row's loads are issued before the current row's arithmetic), the
// statistics need shuffles only and no barrier is met inside the loop.  gamma and beta sit in shared memory as float32,
// laid out so that a lane's 16-byte reads are conflict-free.  Summation order = the thread-group kernel's with "vector j
// of lane l" in the place of "warp j of the group" (the order residual_layernorm_kernel uses as well), so both kernels
// and the CPU oracle agree bit for bit.  FULL: the row fills its NV x 32 vectors exactly (no column guards).  A row
// length that is a power of two divides the sums by multiplying with its exact reciprocal (the same float32 result).
// Used for rows of at least 32 vectors; the thread-group kernel keeps the narrow rows.
template <typename T, int VEC, int NV, bool FULL>
__global__ void __launch_bounds__(kRowWarps * 32, (NV * VEC > 32) ? 1 : 2)  // 64 channels per lane need the whole register file
merge_layernorm_rows_kernel(const T *__restrict__ tokens, const uint8_t *__restrict__ mask, const int *__restrict__ group_prefix,
                            const int *__restrict__ offsets, FrameLayout L, int frames, int Cv, const T *__restrict__ gamma,
                            const T *__restrict__ beta, float eps, T *__restrict__ out) {
    using PIO = PairIO<T, VEC>;
    using V = typename VecIO<T, VEC>::V;
    constexpr int NP = VEC / 2;       // float32 pairs per vector
    constexpr int NQ = (NP + 1) / 2;  // 16-byte chunks of float32 pairs per vector
    // [gamma | beta][vector j of the lane][chunk q][lane] -> 16 bytes = the pairs 2q, 2q + 1 of that vector
    __shared__ __align__(16) f32x2_t s_gb[2][NV][NQ][32][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < NV * 32; i += kRowWarps * 32) {
        const int j = i >> 5, l = i & 31;
        f32x2_t g2[NP], b2[NP];
#pragma unroll
        for (int k = 0; k < NP; ++k) g2[k] = b2[k] = 0ull;
        if (FULL || i < Cv) {
            PIO::unpack(reinterpret_cast<const V *>(gamma)[i], g2);
            PIO::unpack(reinterpret_cast<const V *>(beta)[i], b2);
        }
#pragma unroll
        for (int k = 0; k < NP; ++k) {
            s_gb[0][j][k >> 1][l][k & 1] = g2[k];
            s_gb[1][j][k >> 1][l][k & 1] = b2[k];
        }
    }
    __syncthreads();
    const int G = L.G;
    const int prefix_units = (L.prefix + G - 1) / G;
    const int units_per_frame = prefix_units + L.M;
    const int n_units = frames * units_per_frame;
    const int C = Cv * VEC;
    const float fC = (float)C, fG = (float)G;
    const bool pow2 = (C & (C - 1)) == 0;
    const float inv_c = 1.0f / fC;  // exact when C is a power of two
    auto over_c = [&](float t) { return pow2 ? __fmul_rn(t, inv_c) : __fdiv_rn(t, fC); };
    auto has = [&](int j) { return FULL || j * 32 + lane < Cv; };

    for (int u = blockIdx.x * kRowWarps + warp; u < n_units; u += gridDim.x * kRowWarps) {
        const int bfr = u / units_per_frame, unit = u - bfr * units_per_frame;
        const int base = offsets[bfr];
        int r0, rows, dst;
        bool merged = false;
        if (unit < prefix_units) {
            r0 = unit * G;
            rows = min(G, L.prefix - r0);
            dst = base + r0;
        } else {
            const int m = unit - prefix_units;
            r0 = L.prefix + m * G;
            rows = G;
            dst = base + L.prefix + group_prefix[(size_t)bfr * L.M + m];
            merged = mask[(size_t)bfr * L.M + m] != 0;
        }
        const int my_src = lane < rows ? L.src_token(r0 + lane) : 0;  // lane r knows where row r of the unit lives
        const V *src_base = reinterpret_cast<const V *>(tokens) + (int64_t)bfr * L.N * Cv;
        V *dst_base = reinterpret_cast<V *>(out) + (int64_t)dst * Cv;
        auto load_row = [&](int r, V (&raw)[NV]) {
            const V *row = src_base + (int64_t)__shfl_sync(0xffffffffu, my_src, r) * Cv;
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (has(j)) raw[j] = ld_stream(row + j * 32 + lane);
        };
        V raw[NV];
        load_row(0, raw);
        f32x2_t acc[NV][NP];
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
            for (int k = 0; k < NP; ++k) acc[j][k] = 0ull;
        for (int r = 0; r < rows; ++r) {
            f32x2_t d[NV][NP];
            float total = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float part = 0.0f;
                if (has(j)) {
                    PIO::unpack(raw[j], d[j]);
                    f32x2_t a = d[j][0];
#pragma unroll
                    for (int k = 1; k < NP; ++k) a = add_f32x2(a, d[j][k]);
                    float even, odd;
                    unpack_f32x2(a, even, odd);
                    part = __fadd_rn(even, odd);
                }
                total = (j == 0) ? part : __fadd_rn(total, part);
            }
            if (r + 1 < rows) load_row(r + 1, raw);  // the next row is on its way while this one is normalised
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, m));
            const float mean = over_c(total);
            const f32x2_t neg_mean = pack_f32x2(-mean, -mean);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float part = 0.0f;
                if (has(j)) {
#pragma unroll
                    for (int k = 0; k < NP; ++k) d[j][k] = add_f32x2(d[j][k], neg_mean);
                    f32x2_t a = mul_f32x2(d[j][0], d[j][0]);
#pragma unroll
                    for (int k = 1; k < NP; ++k) a = fma_f32x2(d[j][k], d[j][k], a);  // explicit: never a separate mul + add
                    float even, odd;
                    unpack_f32x2(a, even, odd);
                    part = __fadd_rn(even, odd);
                }
                total = (j == 0) ? part : __fadd_rn(total, part);
            }
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, m));
            const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(over_c(total), eps)));
            const f32x2_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (has(j)) {
                    const int v = j * 32 + lane;
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        const ulonglong2 g = *reinterpret_cast<const ulonglong2 *>(&s_gb[0][j][q][lane][0]);
                        const ulonglong2 b = *reinterpret_cast<const ulonglong2 *>(&s_gb[1][j][q][lane][0]);
                        d[j][2 * q] = fma_f32x2(g.x, mul_f32x2(rstd2, d[j][2 * q]), b.x);
                        if (2 * q + 1 < NP) d[j][2 * q + 1] = fma_f32x2(g.y, mul_f32x2(rstd2, d[j][2 * q + 1]), b.y);
                    }
                    if (merged) {
                        // the normalised tensor lives in T: its rounded values are what the window mean sums
#pragma unroll
                        for (int k = 0; k < NP; ++k) acc[j][k] = add_f32x2(acc[j][k], PIO::round_pair(d[j][k]));
                    } else {
                        st_stream(dst_base + (int64_t)r * Cv + v, PIO::pack(d[j]));
                    }
                }
            }
        }
        if (merged) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (has(j)) {
#pragma unroll
                    for (int k = 0; k < NP; ++k) {
                        float lo, hi;
                        unpack_f32x2(acc[j][k], lo, hi);
                        acc[j][k] = pack_f32x2(__fdiv_rn(lo, fG), __fdiv_rn(hi, fG));
                    }
                    st_stream(dst_base + j * 32 + lane, PIO::pack(acc[j]));
                }
            }
        }
    }
}

template <typename T>
static int launch_merge_layernorm(const void *tokens, int64_t frames, int64_t C, const FrameLayout &L, const uint8_t *mask,
                                  const int32_t *gp, const int32_t *off, const void *gamma, const void *beta, float eps,
                                  void *out, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const auto al = [](const void *p) { return (uintptr_t)p % 16 == 0; };
    if (C % VEC != 0 || C / VEC > kMergeThreads || !al(tokens) || !al(out) || !al(gamma) || !al(beta) || L.G > kLnMaxRows) {
        set_error("come_merge_layernorm needs 16-byte aligned tensors, channels a multiple of %d and at most %d, group size <= %d "
                  "(got channels %lld, group size %d)", VEC, VEC * kMergeThreads, kLnMaxRows, (long long)C, L.G);
        return COME_ERR_UNSUPPORTED;
    }
    const int Cv = (int)(C / VEC);
    int tpg = 32;
    while (tpg < Cv) tpg <<= 1;
    const int groups = kMergeThreads / tpg;
    const int prefix_units = (L.prefix + L.G - 1) / L.G;
    const int64_t n_units = frames * (int64_t)(prefix_units + L.M);
    if (n_units == 0) return COME_OK;
    if (Cv >= 32 && !ln_rows_disabled()) {  // a warp per unit: no barriers, the next row's loads behind the current row's arithmetic
        int64_t blocks = (n_units + kRowWarps - 1) / kRowWarps;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (blocks > cap) blocks = cap;
#define COME_LNR_LAUNCH(NV)                                                                                             \
    do {                                                                                                                \
        if (Cv == 32 * (NV))                                                                                            \
            merge_layernorm_rows_kernel<T, VEC, NV, true><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(                 \
                (const T *)tokens, mask, gp, off, L, (int)frames, Cv, (const T *)gamma, (const T *)beta, eps, (T *)out); \
        else                                                                                                            \
            merge_layernorm_rows_kernel<T, VEC, NV, false><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(                \
                (const T *)tokens, mask, gp, off, L, (int)frames, Cv, (const T *)gamma, (const T *)beta, eps, (T *)out); \
    } while (0)
        if (Cv <= 32) COME_LNR_LAUNCH(1);
        else if (Cv <= 64) COME_LNR_LAUNCH(2);
        else if (Cv <= 128) COME_LNR_LAUNCH(4);
        else COME_LNR_LAUNCH(8);
#undef COME_LNR_LAUNCH
        return check_launch("come_merge_layernorm");
    }
    const size_t smem = (size_t)groups * L.G * sizeof(int) + (size_t)groups * kLnMaxRows * (tpg + 1) * sizeof(float);
    const int64_t n_ctas = (n_units + groups - 1) / groups;
    const int64_t max_blocks = (int64_t)sm_count() * 8;
    const unsigned grid = (unsigned)(n_ctas < max_blocks ? n_ctas : max_blocks);
#define COME_LN_LAUNCH(TPG)                                                                                            \
    merge_layernorm_kernel<T, VEC, TPG><<<grid, kMergeThreads, smem, st>>>((const T *)tokens, mask, gp, off, L, (int)frames, Cv, \
                                                                           groups, (const T *)gamma, (const T *)beta, eps, (T *)out)
    switch (Cv == tpg ? tpg : 0) {  // rows that fill their thread group exactly take a compile-time group size
        case 32: COME_LN_LAUNCH(32); break;
        case 64: COME_LN_LAUNCH(64); break;
        case 128: COME_LN_LAUNCH(128); break;
        case 256: COME_LN_LAUNCH(256); break;
        default: COME_LN_LAUNCH(0); break;
    }
#undef COME_LN_LAUNCH
    return check_launch("come_merge_layernorm");
}

extern "C" int come_merge_layernorm(const void *tokens_dev, int dtype, int64_t frames, int64_t channels,
                                    const come_layout_t *layout, const void *gamma_dev, const void *beta_dev, float eps,
                                    const uint8_t *mask_dev, const int32_t *group_prefix_dev, const int32_t *offsets_dev,
                                    void *out_dev, void *stream) {
    FrameLayout L;
    int rc = make_layout(layout, &L);
    if (rc != COME_OK) return rc;
    COME_REQUIRE(frames >= 0 && channels >= 0, "frames and channels must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(frames * (int64_t)L.N < (1ll << 31), "frames * tokens_per_frame must fit int32 row indices");
    if (frames == 0 || channels == 0) return COME_OK;
    COME_REQUIRE(tokens_dev && out_dev && offsets_dev && gamma_dev && beta_dev, "tokens / out / offsets / gamma / beta must not be NULL");
    COME_REQUIRE(L.M == 0 || (mask_dev && group_prefix_dev), "mask / group_prefix must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case COME_F32: return launch_merge_layernorm<float>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, gamma_dev, beta_dev, eps, out_dev, st);
        case COME_F16: return launch_merge_layernorm<__half>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, gamma_dev, beta_dev, eps, out_dev, st);
        default: return launch_merge_layernorm<__nv_bfloat16>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, gamma_dev, beta_dev, eps, out_dev, st);
    }
}

// ---- unmerge ------------------------------------------------------------------------------------------------------
constexpr int kUnmergeThreads = 256;
constexpr int kUnmergeBatch = 4;

template <typename V>
__global__ void __launch_bounds__(kUnmergeThreads)
unmerge_kernel(const V *__restrict__ merged, const int64_t *__restrict__ rev, int64_t total, int64_t Cv,
               V *__restrict__ out, int64_t out_stride) {
    const int64_t n = total * Cv;
    const int64_t stride = (int64_t)gridDim.x * kUnmergeThreads;
    for (int64_t i0 = (int64_t)blockIdx.x * kUnmergeThreads + threadIdx.x; i0 < n; i0 += stride * kUnmergeBatch) {
        V buf[kUnmergeBatch];
#pragma unroll
        for (int k = 0; k < kUnmergeBatch; ++k) {
            const int64_t i = i0 + k * stride;
            if (i < n) {
                const int64_t row = i / Cv, v = i - row * Cv;
                buf[k] = merged[__ldg(rev + row) * Cv + v];  // merged rows are re-read up to G times: keep in L2
            }
        }
#pragma unroll
        for (int k = 0; k < kUnmergeBatch; ++k) {
            const int64_t i = i0 + k * stride;
            if (i < n) {
                const int64_t row = i / Cv, v = i - row * Cv;
                st_stream(out + row * out_stride + v, buf[k]);
            }
        }
    }
}

// Row-shaped variant for rows of at most 256 vectors that divide 256 (C = 1024 fp32, C = 1024 or 2048 16-bit, ...):
// a CTA moves kRowBatch groups of adjacent output rows per round, one vector per thread and group, with 32-bit index
// arithmetic only (the generic kernel spends a 64-bit division per vector), the row index fetched once per row.
constexpr int kRowBatch = 4;

template <typename V>
__global__ void __launch_bounds__(kUnmergeThreads)
unmerge_rows_kernel(const V *__restrict__ merged, const int64_t *__restrict__ rev, int total, int Cv, V *__restrict__ out,
                    int64_t out_stride) {
    const int rows_per_group = kUnmergeThreads / Cv;
    const int sub = threadIdx.x / Cv, v = threadIdx.x - sub * Cv;
    const int rows_per_round = rows_per_group * kRowBatch;
    for (int row0 = blockIdx.x * rows_per_round; row0 < total; row0 += gridDim.x * rows_per_round) {
        int64_t src[kRowBatch];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            const int row = row0 + k * rows_per_group + sub;
            if (row < total) src[k] = __ldg(rev + row);
        }
        V buf[kRowBatch];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k)
            if (row0 + k * rows_per_group + sub < total) buf[k] = merged[src[k] * Cv + v];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            const int row = row0 + k * rows_per_group + sub;
            if (row < total) st_stream(out + (int64_t)row * out_stride + v, buf[k]);
        }
    }
}

}  // namespace come

// =====================================================================================================================
// C ABI
// =====================================================================================================================
using namespace come;

extern "C" int come_version(void) { return COME_B200_VERSION; }
extern "C" const char *come_last_error(void) { return t_error; }

extern "C" int come_layout_info(const come_layout_t *layout, int64_t *n_groups, int64_t *tokens_per_frame,
                                int64_t *prefix_len) {
    FrameLayout L;
    int rc = make_layout(layout, &L);
    if (rc != COME_OK) return rc;
    if (n_groups) *n_groups = L.M;
    if (tokens_per_frame) *tokens_per_frame = L.N;
    if (prefix_len) *prefix_len = L.prefix;
    return COME_OK;
}

extern "C" size_t come_merge_plan_workspace_bytes(int64_t frames) {
    return (size_t)(frames > 0 ? frames : 1) * sizeof(int);
}

extern "C" int come_merge_plan(const uint8_t *mask_dev, int64_t frames, const come_layout_t *layout,
                               int32_t *group_prefix_dev, int32_t *offsets_dev, int64_t *rev_id_dev,
                               float *weight_dev, int32_t *seg_max_dev, void *workspace_dev, size_t workspace_bytes,
                               void *stream) {
    FrameLayout L;
    int rc = make_layout(layout, &L);
    if (rc != COME_OK) return rc;
    COME_REQUIRE(frames >= 0, "frames must be >= 0");
    COME_REQUIRE(offsets_dev, "offsets must not be NULL");
    COME_REQUIRE(frames == 0 || (int64_t)L.N == 0 || (rev_id_dev && weight_dev), "rev_id / weight must not be NULL");
    COME_REQUIRE(frames == 0 || L.M == 0 || (mask_dev && group_prefix_dev), "mask / group_prefix must not be NULL");
    COME_REQUIRE(frames * (int64_t)L.N < (1ll << 31), "frames * tokens_per_frame must fit int32 row indices");
    COME_REQUIRE(workspace_dev && workspace_bytes >= come_merge_plan_workspace_bytes(frames),
                 "workspace too small: need %zu bytes", come_merge_plan_workspace_bytes(frames));
    cudaStream_t st = (cudaStream_t)stream;
    if (frames == 0) {
        COME_CUDA(cudaMemsetAsync(offsets_dev, 0, sizeof(int32_t), st));
        if (seg_max_dev) COME_CUDA(cudaMemsetAsync(seg_max_dev, 0, sizeof(int32_t), st));
        return COME_OK;
    }
    int *frame_len = (int *)workspace_dev;
    const int warps_per_block = 8;
    plan_count_kernel<<<(unsigned)((frames + warps_per_block - 1) / warps_per_block), warps_per_block * 32, 0, st>>>(
        mask_dev, (int)frames, L.M, L.G, L.prefix, frame_len);
    plan_write_kernel<<<(unsigned)frames, kPlanThreads, 0, st>>>(mask_dev, frame_len, (int)frames, L, group_prefix_dev,
                                                                  offsets_dev, rev_id_dev, weight_dev, seg_max_dev);
    return check_launch("come_merge_plan");
}

// ---- allocation-free plan --------------------------------------------------------------------------------------
// Scratch of come_merge_plan_static: one packed frame length per frame.  A __device__ array is part of the
// loaded module, so every GPU that loads the library carries these 16 KiB until the process exits.
static __device__ __align__(256) int g_plan_scratch[COME_MERGE_PLAN_STATIC_MAX_FRAMES];

// Device address of g_plan_scratch on the current device.  In host code the array's name is only a handle; the
// address a kernel can use has to be asked for, once per device, with that device current.
static int *plan_scratch_dev() {
    static int *cached[64];
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice failed or device index out of range: %s", cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        int *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_plan_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("cudaGetSymbolAddress(plan scratch) failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev] = p;
    }
    return cached[dev];
}

extern "C" int come_merge_plan_static(const uint8_t *mask_dev, int64_t frames, const come_layout_t *layout,
                                      int32_t *group_prefix_dev, int32_t *offsets_dev, int64_t *rev_id_dev,
                                      float *weight_dev, int32_t *seg_max_dev, void *stream) {
    COME_REQUIRE(frames <= COME_MERGE_PLAN_STATIC_MAX_FRAMES,
                 "come_merge_plan_static handles at most %d frames per call, got %lld; use come_merge_plan with a "
                 "caller-provided workspace for more",
                 COME_MERGE_PLAN_STATIC_MAX_FRAMES, (long long)frames);
    int *scratch = plan_scratch_dev();
    if (!scratch) return COME_ERR_CUDA;
    // Every entry of the scratch that pass 2 reads is written by pass 1 of the same call: nothing to clear.
    return come_merge_plan(mask_dev, frames, layout, group_prefix_dev, offsets_dev, rev_id_dev, weight_dev, seg_max_dev,
                           scratch, sizeof(int) * COME_MERGE_PLAN_STATIC_MAX_FRAMES, stream);
}

template <typename T>
static int launch_merge(const void *tokens, int64_t frames, int64_t C, const FrameLayout &L, const uint8_t *mask,
                        const int32_t *gp, const int32_t *off, void *out, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const int prefix_units = (L.prefix + L.G - 1) / L.G;
    const int64_t n_units = frames * (int64_t)(prefix_units + L.M);
    if (n_units == 0 || C == 0) return COME_OK;
    const int64_t max_blocks = (int64_t)sm_count() * 8;  // 8 resident CTAs of 256 threads per SM
    const bool vec_ok = (C % VEC == 0) && ((uintptr_t)tokens % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const int64_t cv = vec_ok ? C / VEC : C;  // vectors per row as the launched kernel sees them
    // Wide rows: the shared-memory ring fed by bulk copies (16-byte multiples, at least four units in the ring).
    {
        const size_t row_bytes = (size_t)C * sizeof(T), stage_bytes = (size_t)L.G * row_bytes;
        const size_t budget = 200 * 1024;
        int stages = stage_bytes ? (int)(budget / stage_bytes) : 0;
        if (stages > kBulkMaxStages) stages = kBulkMaxStages;
        // A stage must always be filled by the same producer and drained by the same store lane (unit k belongs to lane
        // k % kBulkLanes and sits in stage k % stages): a parity wait is only valid for a waiter that is at most one phase
        // behind its barrier, and two lanes taking turns on a stage are not ordered against each other.
        stages -= stages % kBulkLanes;
        const bool aligned = ((uintptr_t)tokens % 16 == 0) && ((uintptr_t)out % 16 == 0) && row_bytes % 16 == 0;
        // Few units per CTA (an 8-frame scene) with rows under 4 KB: the ring's fill and drain cost more than it returns
        // (bfloat16, 8 frames: 11.9 us against 8.3 us of merge_kernel; 100 frames: 76.7 against 81.8 us; float32 wins at both).
        const bool few_small = n_units < 16 * (int64_t)sm_count() && row_bytes < 4096;
        if (vec_ok && aligned && stages >= 4 && row_bytes >= 512 && L.G <= 32 && !few_small && !bulk_disabled()) {
            unsigned int *status = status_word_dev();
            if (!status) return COME_ERR_CUDA;
            const size_t smem_bulk = (size_t)stages * stage_bytes + (size_t)stages * (2 * sizeof(uint64_t) + sizeof(BulkUnit)) + 16;
            int rc = ensure_bulk_smem<T, VEC>(smem_bulk);
            if (rc != COME_OK) return rc;
            const int sms = sm_count();
            const unsigned grid_b = (unsigned)(n_units < sms ? n_units : sms);
            merge_bulk_kernel<T, VEC><<<grid_b, kBulkThreads, smem_bulk, st>>>((const T *)tokens, mask, gp, off, L, (int)frames, C, stages,
                                                                                (T *)out, status);
            return check_launch("come_merge (bulk ring)");
        }
    }
    int groups = 1;
    if (cv >= 32 && cv < kMergeThreads && kMergeThreads % cv == 0) groups = (int)(kMergeThreads / cv);
    while (groups > 1 && (size_t)L.G * sizeof(int) * groups > 48 * 1024) groups >>= 1;
    const size_t smem = (size_t)L.G * sizeof(int) * (size_t)groups;
    const int64_t n_ctas = (n_units + groups - 1) / groups;
    const unsigned grid = (unsigned)(n_ctas < max_blocks ? n_ctas : max_blocks);
    const bool small = n_ctas <= (int64_t)sm_count() * 6;  // at most ~three waves of the two-CTA-per-SM variant
    if (vec_ok && small)
        merge_kernel<T, VEC, 5, 4><<<grid, kMergeThreads, smem, st>>>((const T *)tokens, mask, gp, off, L, (int)frames, C, groups, (T *)out);
    else if (vec_ok)
        merge_kernel<T, VEC, kMaxInFlight, 2><<<grid, kMergeThreads, smem, st>>>((const T *)tokens, mask, gp, off, L, (int)frames, C, groups, (T *)out);
    else
        merge_kernel<T, 1, kMaxInFlight, 2><<<grid, kMergeThreads, smem, st>>>((const T *)tokens, mask, gp, off, L, (int)frames, C, groups, (T *)out);
    return check_launch("come_merge");
}

extern "C" int come_merge(const void *tokens_dev, int dtype, int64_t frames, int64_t channels,
                          const come_layout_t *layout, const uint8_t *mask_dev, const int32_t *group_prefix_dev,
                          const int32_t *offsets_dev, void *out_dev, void *stream) {
    FrameLayout L;
    int rc = make_layout(layout, &L);
    if (rc != COME_OK) return rc;
    COME_REQUIRE(frames >= 0 && channels >= 0, "frames and channels must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE((size_t)L.G * sizeof(int) <= 48 * 1024, "group_size %d too large", L.G);
    COME_REQUIRE(frames * (int64_t)L.N < (1ll << 31), "frames * tokens_per_frame must fit int32 row indices");
    if (frames == 0 || channels == 0) return COME_OK;
    COME_REQUIRE(tokens_dev && out_dev && offsets_dev, "tokens / out / offsets must not be NULL");
    COME_REQUIRE(L.M == 0 || (mask_dev && group_prefix_dev), "mask / group_prefix must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case COME_F32: return launch_merge<float>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, out_dev, st);
        case COME_F16: return launch_merge<__half>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, out_dev, st);
        default: return launch_merge<__nv_bfloat16>(tokens_dev, frames, channels, L, mask_dev, group_prefix_dev, offsets_dev, out_dev, st);
    }
}

template <typename V>
static int launch_unmerge(const void *merged, const int64_t *rev, int64_t total, int64_t Cv, void *out, int64_t out_stride,
                          cudaStream_t st) {
    if (Cv <= kUnmergeThreads && kUnmergeThreads % Cv == 0 && total < (1ll << 31)) {
        const int rows_per_round = (kUnmergeThreads / (int)Cv) * kRowBatch;
        int64_t blocks = (total + rows_per_round - 1) / rows_per_round;
        const int64_t max_blocks = (int64_t)sm_count() * 8;
        if (blocks > max_blocks) blocks = max_blocks;
        unmerge_rows_kernel<V><<<(unsigned)blocks, kUnmergeThreads, 0, st>>>((const V *)merged, rev, (int)total, (int)Cv, (V *)out, out_stride);
        return check_launch("come_unmerge");
    }
    const int64_t n = total * Cv;
    const int64_t per_block = (int64_t)kUnmergeThreads * kUnmergeBatch;
    int64_t blocks = (n + per_block - 1) / per_block;
    const int64_t max_blocks = (int64_t)sm_count() * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    unmerge_kernel<V><<<(unsigned)blocks, kUnmergeThreads, 0, st>>>((const V *)merged, rev, total, Cv, (V *)out, out_stride);
    return check_launch("come_unmerge");
}

// ---- unmerge fused with the block's residual update -----------------------------------------------------------------
// out[i, :] = residual[i, :] + scale[:] * merged[rev[i], :], evaluated like the tensor expression in the element type:
// the product is rounded to T (skipped without a scale), then the sum is rounded to T.
template <typename T, int VEC>
__device__ __forceinline__ typename VecIO<T, VEC>::V residual_update(const typename VecIO<T, VEC>::V &u,
                                                                      const typename VecIO<T, VEC>::V &r, const float (&g)[VEC],
                                                                      bool has_scale) {
    using IO = VecIO<T, VEC>;
    float fu[VEC], fr[VEC];
    IO::unpack(u, fu);
    IO::unpack(r, fr);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        float t = fu[i];
        if (has_scale) t = Elem<T>::to_f32(Elem<T>::from_f32(__fmul_rn(t, g[i])));
        fr[i] = __fadd_rn(fr[i], t);
    }
    return IO::pack(fr);
}

// Rows of at most 256 vectors whose count divides 256: a thread keeps its column (and its slice of the scale) for all the
// rows it visits; kRowBatch row gathers and residual loads in flight per thread.
template <typename T, int VEC>
__global__ void __launch_bounds__(kUnmergeThreads)
unmerge_residual_rows_kernel(const T *__restrict__ merged, const int64_t *__restrict__ rev, int total, int Cv,
                             const T *__restrict__ residual, const T *__restrict__ scale, T *__restrict__ out) {
    using IO = VecIO<T, VEC>;
    using V = typename IO::V;
    const V *m = reinterpret_cast<const V *>(merged);
    const V *res = reinterpret_cast<const V *>(residual);
    V *o = reinterpret_cast<V *>(out);
    const int rows_per_group = kUnmergeThreads / Cv;
    const int sub = threadIdx.x / Cv, v = threadIdx.x - sub * Cv;
    const int rows_per_round = rows_per_group * kRowBatch;
    float g[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) g[i] = 1.0f;
    if (scale) IO::unpack(reinterpret_cast<const V *>(scale)[v], g);
    for (int row0 = blockIdx.x * rows_per_round; row0 < total; row0 += gridDim.x * rows_per_round) {
        int64_t src[kRowBatch];
        V r[kRowBatch], u[kRowBatch];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            const int row = row0 + k * rows_per_group + sub;
            if (row < total) {
                src[k] = __ldg(rev + row);
                r[k] = ld_stream(res + (int64_t)row * Cv + v);
            }
        }
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k)
            if (row0 + k * rows_per_group + sub < total) u[k] = m[src[k] * Cv + v];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            const int row = row0 + k * rows_per_group + sub;
            if (row < total) st_stream(o + (int64_t)row * Cv + v, residual_update<T, VEC>(u[k], r[k], g, scale != nullptr));
        }
    }
}

// Any row width (and the scalar path for unaligned pointers): flat loop over the vectors of the output.
template <typename T, int VEC>
__global__ void __launch_bounds__(kUnmergeThreads)
unmerge_residual_kernel(const T *__restrict__ merged, const int64_t *__restrict__ rev, int64_t total, int64_t Cv,
                        const T *__restrict__ residual, const T *__restrict__ scale, T *__restrict__ out) {
    using IO = VecIO<T, VEC>;
    using V = typename IO::V;
    const V *m = reinterpret_cast<const V *>(merged);
    const V *res = reinterpret_cast<const V *>(residual);
    V *o = reinterpret_cast<V *>(out);
    const int64_t n = total * Cv;
    for (int64_t i = (int64_t)blockIdx.x * kUnmergeThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kUnmergeThreads) {
        const int64_t row = i / Cv, v = i - row * Cv;
        float g[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[k] = 1.0f;
        if (scale) IO::unpack(reinterpret_cast<const V *>(scale)[v], g);
        st_stream(o + i, residual_update<T, VEC>(m[__ldg(rev + row) * Cv + v], ld_stream(res + i), g, scale != nullptr));
    }
}

template <typename T>
static int launch_unmerge_residual(const void *merged, const int64_t *rev, int64_t total, int64_t C, const void *residual,
                                   const void *scale, void *out, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const auto al = [](const void *p) { return (uintptr_t)p % 16 == 0; };
    const bool vec_ok = C % VEC == 0 && al(merged) && al(residual) && al(out) && (!scale || al(scale));
    const int64_t Cv = vec_ok ? C / VEC : C;
    const int64_t max_blocks = (int64_t)sm_count() * 8;
    if (vec_ok && Cv <= kUnmergeThreads && kUnmergeThreads % Cv == 0 && total < (1ll << 31)) {
        const int rows_per_round = (kUnmergeThreads / (int)Cv) * kRowBatch;
        int64_t blocks = (total + rows_per_round - 1) / rows_per_round;
        if (blocks > max_blocks) blocks = max_blocks;
        unmerge_residual_rows_kernel<T, VEC><<<(unsigned)blocks, kUnmergeThreads, 0, st>>>(
            (const T *)merged, rev, (int)total, (int)Cv, (const T *)residual, (const T *)scale, (T *)out);
        return check_launch("come_unmerge_residual");
    }
    int64_t blocks = (total * Cv + kUnmergeThreads - 1) / kUnmergeThreads;
    if (blocks > max_blocks) blocks = max_blocks;
    if (vec_ok)
        unmerge_residual_kernel<T, VEC><<<(unsigned)blocks, kUnmergeThreads, 0, st>>>(
            (const T *)merged, rev, total, Cv, (const T *)residual, (const T *)scale, (T *)out);
    else
        unmerge_residual_kernel<T, 1><<<(unsigned)blocks, kUnmergeThreads, 0, st>>>(
            (const T *)merged, rev, total, Cv, (const T *)residual, (const T *)scale, (T *)out);
    return check_launch("come_unmerge_residual");
}

extern "C" int come_unmerge_residual(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels,
                                     int dtype, const void *residual_dev, const void *scale_dev, void *out_dev,
                                     void *stream) {
    COME_REQUIRE(total >= 0 && channels >= 0, "total and channels must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    if (total == 0 || channels == 0) return COME_OK;
    COME_REQUIRE(merged_dev && rev_id_dev && residual_dev && out_dev, "merged / rev_id / residual / out must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case COME_F32: return launch_unmerge_residual<float>(merged_dev, rev_id_dev, total, channels, residual_dev, scale_dev, out_dev, st);
        case COME_F16: return launch_unmerge_residual<__half>(merged_dev, rev_id_dev, total, channels, residual_dev, scale_dev, out_dev, st);
        default: return launch_unmerge_residual<__nv_bfloat16>(merged_dev, rev_id_dev, total, channels, residual_dev, scale_dev, out_dev, st);
    }
}

// ---- residual update fused with the LayerNorm behind it (packed rows, no gather) --------------------------------------
// x_out = x + scale * branch  (LayerScale and the residual add that close a sub-block; each tensor operation rounded to T)
// normed = LayerNorm(x_out)   (the norm that opens the next sub-block)
// One warp owns a row: lane l holds the 16-byte vectors l, l + 32, ... of the row (NV of them), so both tensors are read
// once, statistics need shuffles only and no barrier is met.  Summation order of the statistics = the fused LayerNorm +
// merge kernel's with "vector j of lane l" in the place of "warp j of the thread group": inside a vector the even / odd
// chains, vectors of a lane left to right, then a butterfly over the lanes (neighbours first).

template <typename T, int VEC, int NV>
__global__ void __launch_bounds__(kRowWarps * 32, NV >= 8 ? 1 : (NV >= 4 ? 2 : 3))  // a row's float32 copy stays in registers
residual_layernorm_kernel(const T *__restrict__ x, const T *__restrict__ branch, const T *__restrict__ scale, int rows, int Cv,
                          const T *__restrict__ gamma, const T *__restrict__ beta, float eps, T *__restrict__ x_out,
                          T *__restrict__ normed) {
    using IO = VecIO<T, VEC>;
    using PIO = PairIO<T, VEC>;
    using V = typename IO::V;
    constexpr int NP = VEC / 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float fC = (float)(Cv * VEC);
    for (int row = blockIdx.x * kRowWarps + warp; row < rows; row += gridDim.x * kRowWarps) {
        const int64_t base = (int64_t)row * Cv;
        V rx[NV], rb[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int v = j * 32 + lane;
            if (v < Cv) {
                rx[j] = ld_stream(reinterpret_cast<const V *>(x) + base + v);
                if (branch) rb[j] = ld_stream(reinterpret_cast<const V *>(branch) + base + v);
            }
        }
        if (branch) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int v = j * 32 + lane;
                if (v < Cv) {
                    float g[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) g[i] = 1.0f;
                    if (scale) IO::unpack(reinterpret_cast<const V *>(scale)[v], g);
                    rx[j] = residual_update<T, VEC>(rb[j], rx[j], g, scale != nullptr);
                    if (x_out) st_stream(reinterpret_cast<V *>(x_out) + base + v, rx[j]);
                }
            }
        }
        if (!normed) continue;
        f32x2_t d[NV][NP];
        float total = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float part = 0.0f;
#pragma unroll
            for (int k = 0; k < NP; ++k) d[j][k] = 0ull;
            if (j * 32 + lane < Cv) {
                PIO::unpack(rx[j], d[j]);
                f32x2_t acc = d[j][0];
#pragma unroll
                for (int k = 1; k < NP; ++k) acc = add_f32x2(acc, d[j][k]);
                float even, odd;
                unpack_f32x2(acc, even, odd);
                part = __fadd_rn(even, odd);
            }
            total = (j == 0) ? part : __fadd_rn(total, part);
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, m));
        const float mean = __fdiv_rn(total, fC);
        const f32x2_t neg_mean = pack_f32x2(-mean, -mean);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float part = 0.0f;
            if (j * 32 + lane < Cv) {
#pragma unroll
                for (int k = 0; k < NP; ++k) d[j][k] = add_f32x2(d[j][k], neg_mean);
                f32x2_t acc = mul_f32x2(d[j][0], d[j][0]);
#pragma unroll
                for (int k = 1; k < NP; ++k) acc = fma_f32x2(d[j][k], d[j][k], acc);  // explicit: never a separate mul + add
                float even, odd;
                unpack_f32x2(acc, even, odd);
                part = __fadd_rn(even, odd);
            }
            total = (j == 0) ? part : __fadd_rn(total, part);
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, m));
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, fC), eps)));
        const f32x2_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int v = j * 32 + lane;
            if (v < Cv) {
                f32x2_t g2[NP], b2[NP];
                PIO::unpack(__ldg(reinterpret_cast<const V *>(gamma) + v), g2);
                PIO::unpack(__ldg(reinterpret_cast<const V *>(beta) + v), b2);
#pragma unroll
                for (int k = 0; k < NP; ++k) d[j][k] = fma_f32x2(g2[k], mul_f32x2(rstd2, d[j][k]), b2[k]);
                st_stream(reinterpret_cast<V *>(normed) + base + v, PIO::pack(d[j]));
            }
        }
    }
}

template <typename T>
static int launch_residual_layernorm(const void *x, const void *branch, const void *scale, int64_t rows, int64_t C,
                                     const void *gamma, const void *beta, float eps, void *x_out, void *normed, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const auto al = [](const void *p) { return !p || (uintptr_t)p % 16 == 0; };
    if (C % VEC != 0 || C / VEC > 256 || !al(x) || !al(branch) || !al(scale) || !al(gamma) || !al(beta) || !al(x_out) || !al(normed)) {
        set_error("come_residual_layernorm needs 16-byte aligned tensors and channels a multiple of %d, at most %d (got %lld)",
                  VEC, VEC * 256, (long long)C);
        return COME_ERR_UNSUPPORTED;
    }
    const int Cv = (int)(C / VEC);
    int64_t blocks = (rows + kRowWarps - 1) / kRowWarps;
    const int64_t max_blocks = (int64_t)sm_count() * 6;  // a few resident waves, then the grid strides
    if (blocks > max_blocks) blocks = max_blocks;
#define COME_RLN_LAUNCH(NV)                                                                                                  \
    residual_layernorm_kernel<T, VEC, NV><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(                                       \
        (const T *)x, (const T *)branch, (const T *)scale, (int)rows, Cv, (const T *)gamma, (const T *)beta, eps, (T *)x_out, (T *)normed)
    if (Cv <= 32) COME_RLN_LAUNCH(1);
    else if (Cv <= 64) COME_RLN_LAUNCH(2);
    else if (Cv <= 128) COME_RLN_LAUNCH(4);
    else COME_RLN_LAUNCH(8);
#undef COME_RLN_LAUNCH
    return check_launch("come_residual_layernorm");
}

extern "C" int come_residual_layernorm(const void *x_dev, const void *branch_dev, const void *scale_dev, int64_t rows,
                                       int64_t channels, int dtype, const void *gamma_dev, const void *beta_dev, float eps,
                                       void *x_out_dev, void *normed_dev, void *stream) {
    COME_REQUIRE(rows >= 0 && channels >= 0, "rows and channels must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(rows < (1ll << 31), "rows must fit int32");
    if (rows == 0 || channels == 0) return COME_OK;
    COME_REQUIRE(x_dev != nullptr, "x must not be NULL");
    COME_REQUIRE(branch_dev || !scale_dev, "scale without a branch");
    COME_REQUIRE(!branch_dev || x_out_dev || normed_dev, "nothing to write");
    COME_REQUIRE(!normed_dev || (gamma_dev && beta_dev), "gamma / beta must not be NULL when normed is requested");
    COME_REQUIRE(branch_dev || normed_dev, "without a branch there is only the LayerNorm to compute: normed must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case COME_F32: return launch_residual_layernorm<float>(x_dev, branch_dev, scale_dev, rows, channels, gamma_dev, beta_dev, eps, x_out_dev, normed_dev, st);
        case COME_F16: return launch_residual_layernorm<__half>(x_dev, branch_dev, scale_dev, rows, channels, gamma_dev, beta_dev, eps, x_out_dev, normed_dev, st);
        default: return launch_residual_layernorm<__nv_bfloat16>(x_dev, branch_dev, scale_dev, rows, channels, gamma_dev, beta_dev, eps, x_out_dev, normed_dev, st);
    }
}

extern "C" int come_unmerge_strided(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels,
                                    int dtype, void *out_dev, int64_t out_row_stride, void *stream) {
    COME_REQUIRE(total >= 0 && channels >= 0, "total and channels must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(out_row_stride >= channels, "out_row_stride (%lld) must be >= channels (%lld)", (long long)out_row_stride,
                 (long long)channels);
    if (total == 0 || channels == 0) return COME_OK;
    COME_REQUIRE(merged_dev && rev_id_dev && out_dev, "merged / rev_id / out must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = dtype_size(dtype);
    const size_t row_bytes = (size_t)channels * es, stride_bytes = (size_t)out_row_stride * es;
    const uintptr_t m = (uintptr_t)merged_dev, o = (uintptr_t)out_dev;
    if (row_bytes % 16 == 0 && stride_bytes % 16 == 0 && m % 16 == 0 && o % 16 == 0)
        return launch_unmerge<uint4>(merged_dev, rev_id_dev, total, row_bytes / 16, out_dev, stride_bytes / 16, st);
    if (row_bytes % 4 == 0 && stride_bytes % 4 == 0 && m % 4 == 0 && o % 4 == 0)
        return launch_unmerge<uint32_t>(merged_dev, rev_id_dev, total, row_bytes / 4, out_dev, stride_bytes / 4, st);
    return launch_unmerge<uint16_t>(merged_dev, rev_id_dev, total, row_bytes / 2, out_dev, stride_bytes / 2, st);
}

extern "C" int come_unmerge(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels,
                            int dtype, void *out_dev, void *stream) {
    return come_unmerge_strided(merged_dev, rev_id_dev, total, channels, dtype, out_dev, channels, stream);
}

// ---- suffix tokens of jagged segments ---------------------------------------------------------------------------------
// add: every segment of a packed sequence gets T dense rows appended (weight 1); split: the inverse.  Segment m of the longer
// sequence starts at offset[m] + m * T, so neither direction needs the other's offsets in memory.  One warp per output row:
// every lane finds the row's segment by the same binary search over the M + 1 offsets (they stay in L1), then the lanes copy the
// row's vectors, four loads in flight each.
template <typename V, bool SPLIT>
__global__ void __launch_bounds__(kRowWarps * 32)
suffix_rows_kernel(const V *__restrict__ tokens, const float *__restrict__ weight, const int64_t *__restrict__ offset, int segments,
                   int64_t rows_out, int Cv, int T, const V *__restrict__ suffix_in, V *__restrict__ out_tokens,
                   float *__restrict__ out_weight, int64_t *__restrict__ out_offset, V *__restrict__ suffix_out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * kRowWarps;
    // offsets of the result: longer by m * T (add) or shorter by m * T (split)
    for (int64_t i = warp * 32 + lane; i <= segments; i += n_warps * 32) out_offset[i] = offset[i] + (SPLIT ? -i : i) * (int64_t)T;
    const int64_t shift = SPLIT ? -(int64_t)T : (int64_t)T;  // out_start(m) = offset[m] + m * shift
    // rows of the packed result, then (split only) the segments x T suffix rows
    const int64_t n_rows = rows_out + (SPLIT ? (int64_t)segments * T : 0);
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        const V *src;
        V *dst;
        float w = 1.0f;
        bool has_w = false;
        if (r < rows_out) {
            int lo = 0, hi = segments;  // the segment with out_start(lo) <= r < out_start(lo + 1)
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (__ldg(offset + mid) + mid * shift <= r) lo = mid;
                else hi = mid;
            }
            const int64_t seg_begin = __ldg(offset + lo), local = r - (seg_begin + lo * shift);
            dst = out_tokens + r * Cv;
            has_w = true;
            if (SPLIT) {  // row `local` of segment lo, whose old rows are all kept up to the new length
                src = tokens + (seg_begin + local) * Cv;
                w = __ldg(weight + seg_begin + local);
            } else {
                const int64_t old_len = __ldg(offset + lo + 1) - seg_begin;
                if (local < old_len) {
                    src = tokens + (seg_begin + local) * Cv;
                    w = __ldg(weight + seg_begin + local);
                } else {
                    src = suffix_in + ((int64_t)lo * T + (local - old_len)) * Cv;
                }
            }
        } else {  // split: suffix row t of segment m = the row T - t before the segment's old end
            const int64_t k = r - rows_out;
            const int m = (int)(k / T), t = (int)(k - (int64_t)m * T);
            src = tokens + (__ldg(offset + m + 1) - T + t) * Cv;
            dst = suffix_out + k * Cv;
        }
        if (has_w && lane == 0) out_weight[r] = w;
        for (int v0 = lane; v0 < Cv; v0 += 128) {
            V tmp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + 32 * j < Cv) tmp[j] = ld_stream(src + v0 + 32 * j);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + 32 * j < Cv) st_stream(dst + v0 + 32 * j, tmp[j]);
        }
    }
}

template <typename V, bool SPLIT>
static int launch_suffix(const void *tokens, const float *weight, const int64_t *offset, int64_t segments, int64_t rows_out,
                         int64_t Cv, int64_t T, const void *suffix_in, void *out_tokens, float *out_weight, int64_t *out_offset,
                         void *suffix_out, cudaStream_t st) {
    const int64_t n_rows = rows_out + (SPLIT ? segments * T : 0);
    int64_t blocks = ((n_rows > segments + 1 ? n_rows : segments / 32 + 1) + kRowWarps - 1) / kRowWarps;
    const int64_t max_blocks = (int64_t)sm_count() * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    if (blocks < 1) blocks = 1;
    suffix_rows_kernel<V, SPLIT><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(
        (const V *)tokens, weight, offset, (int)segments, rows_out, (int)Cv, (int)T, (const V *)suffix_in, (V *)out_tokens, out_weight,
        out_offset, (V *)suffix_out);
    return check_launch(SPLIT ? "come_suffix_split" : "come_suffix_add");
}

template <bool SPLIT>
static int suffix_dispatch(const void *tokens, const float *weight, const int64_t *offset, int64_t segments, int64_t total,
                           int64_t channels, int dtype, int64_t T, const void *suffix_in, void *out_tokens, float *out_weight,
                           int64_t *out_offset, void *suffix_out, void *stream) {
    COME_REQUIRE(segments >= 0 && total >= 0 && channels >= 0 && T >= 0, "segments, total, channels and suffix_len must be >= 0");
    COME_REQUIRE(dtype == COME_F32 || dtype == COME_F16 || dtype == COME_BF16, "unknown dtype %d", dtype);
    COME_REQUIRE(segments < (1ll << 31) && T < (1ll << 31), "segments and suffix_len must fit int32");
    COME_REQUIRE(offset && out_offset, "offset / out_offset must not be NULL");
    COME_REQUIRE(segments > 0 || total == 0, "tokens without segments");
    const int64_t rows_out = SPLIT ? total - segments * T : total + segments * T;
    COME_REQUIRE(rows_out >= 0, "cannot strip %lld tokens from each of %lld segments (total tokens = %lld)", (long long)T,
                 (long long)segments, (long long)total);
    const bool moves = channels > 0 && (rows_out > 0 || (SPLIT && segments * T > 0));
    COME_REQUIRE(!moves || (tokens || total == 0), "tokens must not be NULL");
    COME_REQUIRE(rows_out == 0 || (out_weight && (weight || total == 0)), "weight / out_weight must not be NULL");
    COME_REQUIRE(!moves || rows_out == 0 || out_tokens, "out_tokens must not be NULL");
    COME_REQUIRE(!moves || segments * T == 0 || (SPLIT ? suffix_out != nullptr : suffix_in != nullptr), "suffix must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t row_bytes = (size_t)channels * dtype_size(dtype);
    const auto al = [](const void *p, size_t a) { return (uintptr_t)p % a == 0; };
    const void *sfx = SPLIT ? suffix_out : suffix_in;
    if (row_bytes % 16 == 0 && al(tokens, 16) && al(out_tokens, 16) && al(sfx, 16))
        return launch_suffix<uint4, SPLIT>(tokens, weight, offset, segments, rows_out, row_bytes / 16, T, suffix_in, out_tokens, out_weight, out_offset, suffix_out, st);
    if (row_bytes % 4 == 0 && al(tokens, 4) && al(out_tokens, 4) && al(sfx, 4))
        return launch_suffix<uint32_t, SPLIT>(tokens, weight, offset, segments, rows_out, row_bytes / 4, T, suffix_in, out_tokens, out_weight, out_offset, suffix_out, st);
    return launch_suffix<uint16_t, SPLIT>(tokens, weight, offset, segments, rows_out, row_bytes / 2, T, suffix_in, out_tokens, out_weight, out_offset, suffix_out, st);
}

extern "C" int come_suffix_add(const void *tokens_dev, const float *weight_dev, const int64_t *offset_dev, int64_t segments,
                               int64_t total, int64_t channels, int dtype, const void *suffix_dev, int64_t suffix_len,
                               void *out_tokens_dev, float *out_weight_dev, int64_t *out_offset_dev, void *stream) {
    return suffix_dispatch<false>(tokens_dev, weight_dev, offset_dev, segments, total, channels, dtype, suffix_len, suffix_dev,
                                  out_tokens_dev, out_weight_dev, out_offset_dev, nullptr, stream);
}

extern "C" int come_suffix_split(const void *tokens_dev, const float *weight_dev, const int64_t *offset_dev, int64_t segments,
                                 int64_t total, int64_t channels, int dtype, int64_t suffix_len, void *out_tokens_dev,
                                 float *out_weight_dev, int64_t *out_offset_dev, void *suffix_out_dev, void *stream) {
    return suffix_dispatch<true>(tokens_dev, weight_dev, offset_dev, segments, total, channels, dtype, suffix_len, nullptr,
                                 out_tokens_dev, out_weight_dev, out_offset_dev, suffix_out_dev, stream);
}

extern "C" int come_device_status(uint32_t *value, int clear) {
    COME_REQUIRE(value != nullptr, "value is NULL");
    unsigned int v = 0;
    unsigned int *word = come::status_word_dev();
    if (!word) return COME_ERR_CUDA;
    COME_CUDA(cudaDeviceSynchronize());
    COME_CUDA(cudaMemcpy(&v, word, sizeof(v), cudaMemcpyDeviceToHost));
    *value = v;
    if (clear && v != 0) COME_CUDA(cudaMemset(word, 0, sizeof(v)));
    if (v != 0) {
        come::set_error("device status word 0x%08x: %s%s%s%s%s", v, (v & 0x1ffu) ? "a bounded wait of the attention kernel ran out; " : "",
                        (v & 0x8000u) ? "the wait self-test ran; " : "", (v & 0x10000u) ? "a position outside the rotary table was clamped; " : "",
                        (v & 0x20000u) ? "a bounded wait of the bulk-copy merge kernel ran out; " : "",
                        (v & 0x40000u) ? "a wait for the other ranks' key / value rows ran out (come_peer_wait); " : "");
        return COME_ERR_DEVICE;
    }
    return COME_OK;
}
