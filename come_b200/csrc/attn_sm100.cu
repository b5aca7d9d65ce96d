// Variable-length biased attention forward on Blackwell tensor cores (sm_100a): tcgen05.mma with TMEM
// accumulators, TMA-fed 128-byte-swizzled Q/K/V tiles, warp-specialised roles.
//
// Persistent kernel: one CTA per SM walks the work items; a work item is the (up to) three 128-row query tiles of one
// (segment, head), whose keys are walked 64 at a time.  Barrier phases keep counting across items.
//   warps 0-3 / 4-7 / 8-11 : softmax group of query tile 0 / 1 / 2.  Thread r owns score row r (TMEM lane r).  Per key
//                     tile it pulls the 64 scores into registers (S is free for the next Q K^T at once), takes the row
//                     max with 3-input max, then p = exp2(s * scale*log2e - m) in packed float32x2 arithmetic, 5 of 16
//                     exponentials on the FMA pipe (cubic polynomial) instead of the special-function unit, writes p
//                     back to TMEM as 16-bit pairs (the A operand of P V) and rescales the accumulator only when the
//                     running max grew by more than 2^8 (exact: the final normalisation uses the same reference max).
//   warp 12         : producer.  Issues the TMA loads of Q (double-buffered across items), K and V and stages, per key
//                     tile, a "bias slab": a 128-byte-swizzled tile whose first two columns hold bias/scale split into
//                     a high and a low 16-bit part (a large negative number past the segment end, which masks the
//                     ragged tail).
//   warps 13, 14, 15 : MMA issuer of query tile 0 / 1 / 2 (one elected lane issues).  S = Q K^T takes four K=16 steps
//                     over the head dimension plus one K=16 step [1 1 0 ...] x [bias_hi bias_lo 0 ...]^T that adds
//                     the per-key bias inside the tensor core; O += P V reads P from TMEM and V (N-major) from
//                     shared memory.  S(j+1) is issued as soon as the softmax group holds S(j) in registers, P V as
//                     soon as P(j) is staged.
// TMEM columns: S_t [64 t, 64 t + 64), O_t [192 + 64 t, ...), P_t [384 + 32 t, ...), t = 0, 1, 2.
//
// Every wait on an mbarrier is bounded: after ~2^29 clock ticks the waiter raises the CTA's abort flag and the
// library's device status word, every role falls through to the common exit, TMEM is released and the kernel
// returns instead of hanging.
#include "attn_sm100.cuh"

#include <cuda.h>

#include <mutex>
#include <type_traits>

namespace come {

namespace {

constexpr int kTiles = 3;         // query tiles (128 rows each) per CTA and work item, one softmax warpgroup each
constexpr int kBlockM = 128;
constexpr int kBlockN = 64;       // keys per step
constexpr int kHeadDim = 64;
constexpr int kStages = 8;        // K/V ring slots, 8 KiB each
constexpr int kSlabStages = 3;    // bias slab ring slots, 8 KiB each (only two 16-byte chunks per row are used)
constexpr int kProducerWarp = 4 * kTiles;      // warps 0 .. 4*kTiles-1 are the softmax groups
constexpr int kIssuerWarp0 = kProducerWarp + 1;  // one MMA issuer warp per query tile
constexpr int kThreads = 32 * (kIssuerWarp0 + kTiles);  // 512: three softmax warpgroups + one producer / issuer warpgroup
// Launches with this many segments enumerate only the query blocks that exist (a prefix table in shared memory)
constexpr int kMinPrefixSegs = 16, kMaxPrefixSegs = 2048;
constexpr int kQTileBytes = kBlockM * kHeadDim * 2;   // 16384
constexpr int kKvTileBytes = kBlockN * kHeadDim * 2;  // 8192
// Tensor-memory columns: S_t (scores, float32) | O_t (accumulator, float32) | P_t (probabilities, 16-bit pairs)
constexpr uint32_t kTmemS = 0, kTmemO = kTiles * kBlockN, kTmemP = kTmemO + kTiles * kHeadDim;
static_assert(kTmemP + kTiles * (kBlockN / 2) <= 512, "tensor memory holds 512 columns");
static_assert(kThreads % 128 == 0, "setmaxnreg works on whole warpgroups");
static_assert(kMaxPrefixSegs % kThreads == 0, "every thread scans the same number of segments");
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitTicks = 1ll << 29;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// Which of the 16 score pairs of a 32-column quarter take the polynomial exp2 (bit i = pair i); the rest use the
// special-function unit.  5 of 16 balanced the two pipes best in measurements of the two-tile predecessor; with three
// tiles in flight shares from 0 to 6 of 16 measure within 2 % of each other.
#ifndef COME_POLY_MASK
#define COME_POLY_MASK 0x4924u
#endif
constexpr uint32_t kPolyPairs = COME_POLY_MASK;
constexpr float kMasked = -3.0e38f;        // "minus infinity" of a masked key, still finite in bfloat16

// Development builds (-DCOME_ATTN_TRACE) accumulate, per warp, the clocks spent in each kind of wait of the key loop and
// leave them in a device array that come_debug_attn_trace() copies out; normal builds carry none of it.
#ifdef COME_ATTN_TRACE
constexpr int kTraceSlots = 12;
__device__ unsigned long long g_attn_trace[256 * (kThreads / 32) * kTraceSlots];
#define TRACE_DECL() long long tr_acc[kTraceSlots] = {}; long long tr_t = 0; (void)tr_t
#define TRACE_BEGIN() tr_t = clock64()
#define TRACE_END(slot) tr_acc[slot] += clock64() - tr_t
#define TRACE_COUNT(slot, n) tr_acc[slot] += (n)
#define TRACE_STAMP(slot, cond) do { if (cond) tr_acc[slot] = clock64(); } while (0)
#define TRACE_FLUSH()                                                                                          \
    do {                                                                                                       \
        if ((threadIdx.x & 31) == 0 && blockIdx.x < 256)                                                       \
            for (int i__ = 0; i__ < kTraceSlots; ++i__)                                                        \
                g_attn_trace[(blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * kTraceSlots + i__] = (unsigned long long)tr_acc[i__]; \
    } while (0)
#else
#define TRACE_DECL()
#define TRACE_BEGIN()
#define TRACE_END(slot)
#define TRACE_COUNT(slot, n)
#define TRACE_STAMP(slot, cond)
#define TRACE_FLUSH()
#endif

struct SharedStorage {
    alignas(1024) uint8_t q[kTiles][2][kQTileBytes];        // [query tile][buffer]: the next item's Q is loaded ahead
    alignas(1024) uint8_t kv[kStages][kKvTileBytes];
    alignas(1024) uint8_t q_slab[kQTileBytes];              // columns 0,1 = 1.0, rest 0: the A side of the bias step
    alignas(1024) uint8_t k_slab[kSlabStages][kKvTileBytes];  // columns 0,1 = bias/scale (hi, lo): the B side
    alignas(8) uint64_t q_full[kTiles][2];                  // [query tile][buffer]
    uint64_t q_empty[kTiles][2];
    uint64_t q_slab_full;
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t slab_full[kSlabStages];
    uint64_t slab_empty[kSlabStages];
    uint64_t s_full[kTiles];
    uint64_t p_full[kTiles];
    uint64_t o_done[kTiles];
    uint64_t s_empty[kTiles];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    int scan_warp[kThreads / 32];
};
// Launches that use the prefix table get (kMaxPrefixSegs + 1) ints of dynamic shared memory behind SharedStorage:
// table[s] = query blocks of the segments before s (this launch's rows).
constexpr size_t kPrefixTableBytes = sizeof(int) * (kMaxPrefixSegs + 1);

static_assert(sizeof(SharedStorage) + kPrefixTableBytes + 1024 <= 227 * 1024, "shared storage exceeds the 227 KB a CTA may use");

// ---- PTX wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag + the device status word) when it gives up after `limit`
// clock ticks, or when another waiter of the CTA has given up.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                unsigned int *status, uint32_t code, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicOr(status, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, SharedStorage &sh, unsigned int *status,
                                          uint32_t code) {
    return mbar_wait_limit(bar, parity, &sh.abort_flag, status, code, kWaitTicks);
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The issuer warps run their loops in warp-uniform control flow; for a group of instructions (the Q K^T of a key tile
// with its commits, or its P V) one lane is elected once and issues the whole group.  Electing per instruction (every
// lane evaluating the operands, one lane executing) measured 3-5 % slower: an issuer warp shares its scheduler with
// three softmax warps, and every instruction it does not issue shortens the time from "P is staged" to "P V is queued".
__device__ __forceinline__ bool elect_one() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e != 0;
}
__device__ __forceinline__ void tc_commit_1(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_ss_1(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_ts_1(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Makes generic-proxy shared-memory writes of this thread visible to the async proxy (tcgen05.mma operands).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// Row r of a slab (128-byte rows, 128-byte swizzle): logical 16-byte chunk c lives at physical chunk c ^ (r % 8).
// Writes columns 0..7 = {v01 (two 16-bit values), 0 ...} and columns 8..15 = 0; the other chunks are never read.
__device__ __forceinline__ void slab_write_row(uint32_t slab_addr, int r, uint32_t v01) {
    const uint32_t row = slab_addr + (uint32_t)r * 128u;
    st_shared_v4(row + (uint32_t)((0 ^ (r & 7)) << 4), v01, 0u, 0u, 0u);
    st_shared_v4(row + (uint32_t)((1 ^ (r & 7)) << 4), 0u, 0u, 0u, 0u);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for two values on the FMA / integer pipes instead of the special-function unit (which is the bottleneck of
// the head_dim-64 kernel): round-to-nearest range reduction x = n + f, f in [-0.5, 0.5], cubic fit of 2^f (relative
// error 1.0e-4, far below the 16-bit rounding of the probabilities), n added to the exponent field as an integer.
// Inputs below -125 are clamped (the result is then ~2^-125, i.e. zero for all purposes).
__device__ __forceinline__ void exp2_poly_x2(float x0, float x1, float &r0, float &r1) {
    const f32x2_t magic = pack_f32x2(12582912.0f, 12582912.0f);  // 1.5 * 2^23: adding it rounds to an integer
    const f32x2_t neg_magic = pack_f32x2(-12582912.0f, -12582912.0f);
    const f32x2_t minus_one = pack_f32x2(-1.0f, -1.0f);
    const f32x2_t c3 = pack_f32x2(0.05583828315138817f, 0.05583828315138817f);
    const f32x2_t c2 = pack_f32x2(0.2426394820213318f, 0.2426394820213318f);
    const f32x2_t c1 = pack_f32x2(0.6931367516517639f, 0.6931367516517639f);
    const f32x2_t c0 = pack_f32x2(0.9999245405197144f, 0.9999245405197144f);
    const f32x2_t x = pack_f32x2(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
    const f32x2_t t = add_f32x2(x, magic);        // low mantissa bits of t hold n = round(x)
    const f32x2_t n = add_f32x2(t, neg_magic);
    const f32x2_t f = fma_f32x2(n, minus_one, x);
    f32x2_t p = fma_f32x2(c3, f, c2);
    p = fma_f32x2(p, f, c1);
    p = fma_f32x2(p, f, c0);
    float p0, p1, t0, t1;
    unpack_f32x2(p, p0, p1);
    unpack_f32x2(t, t0, t1);
    r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
    r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

template <bool kBF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (kBF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
}

// Multiplies the 64 float32 accumulator columns of this thread's row by alpha (the rare rescale when a row's running
// max grew past the threshold).  Out of line: inlined it would only bloat the hot loop.
__device__ __noinline__ void scale_accumulator(uint32_t o_tmem, float alpha) {
    uint32_t o[2][32];
    tmem_ld32(o_tmem + 0, o[0]);
    tmem_ld32(o_tmem + 32, o[1]);
    tc_wait_ld();
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c][i] = __float_as_uint(__uint_as_float(o[c][i]) * alpha);
    tmem_st32(o_tmem + 0, o[0]);
    tmem_st32(o_tmem + 32, o[1]);
}

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes wide and 128-byte swizzled (what a TMA
// load with a 64-element 16-bit inner box produces): 8-row groups are 1024 bytes apart.  The same encoding
// serves a K-major operand (rows = M/N index, advance 32 bytes per 16-element K step) and an MN-major operand
// (rows = K index, advance 2048 bytes per 16-row K step).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);  // start address
    d |= (uint64_t)1 << 16;                   // leading byte offset (unused for a single swizzle atom)
    d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                   // 128-byte swizzle
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: float32 accumulate, 16-bit A/B of the given format.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, int M, int N, bool b_mn_major) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

enum : uint32_t {
    kErrQFull = 1u << 0, kErrKvFull = 1u << 1, kErrKvEmpty = 1u << 2, kErrSlabFull = 1u << 3, kErrSlabEmpty = 1u << 4,
    kErrSFull = 1u << 5, kErrSEmpty = 1u << 6, kErrPFull = 1u << 7, kErrODone = 1u << 8,
    kErrSelfTest = 1u << 15,  // raised by the wait self-test on purpose
};

// One work item = the (up to) kTiles 128-row query tiles [q_row0, q_row0 + kTiles * 128) of one (segment, head).
struct WorkItem {
    int head, s0, s1;   // head, key range of the segment
    int q_row0, q_hi;   // first query row of the item, end of the query rows this launch owns in the segment
    int n_mt, n_kv;     // active query tiles (1 .. kTiles), key tiles
    bool ragged_tail;   // the last key tile is partial
    bool valid;
    int kpart;          // which share of the keys this item covers (launches that split the keys of their items), else 0
};

// Query blocks of segment `seg` that hold rows of this launch.
__device__ __forceinline__ int segment_blocks(int seg, const int *__restrict__ cu, int q_begin, int q_end) {
    const int rows = min(cu[seg + 1], q_end) - max(cu[seg], q_begin);
    return rows > 0 ? (rows + kTiles * kBlockM - 1) / (kTiles * kBlockM) : 0;
}

// Item -> (head, segment, query block).  With a prefix table (seg_prefix != nullptr) the items are exactly the query
// blocks that exist, in (head, segment, block) order; without it every segment gets `nblk_x` slots and the surplus ones
// are skipped as invalid.
// q_free: the launch has one segment whose keys all query rows [q_begin, q_end) attend to, whether or not those rows lie
// inside the segment (attention of this GPU's rows to keys gathered from other GPUs); cu may then be NULL = [0, kv_total].
template <bool kPrefix>
__device__ __forceinline__ WorkItem decode_item(int item, int nblk_x, int nseg, const int *__restrict__ cu, int q_begin, int q_end,
                                                const int *seg_prefix, int kv_total, bool q_free, int k_parts = 1) {
    WorkItem w;
    int bx, seg;
    // Launches with k_parts > 1 (q_free only): consecutive items are the shares of the key tiles of one (head, block); every
    // share writes its own output and log-sum-exp, merged afterwards.  The host picks k_parts so that no share is empty.
    w.kpart = 0;
    if (k_parts > 1) {
        w.kpart = item % k_parts;
        item /= k_parts;
    }
    if constexpr (kPrefix) {
        const int per_head = seg_prefix[nseg];
        w.head = item / per_head;
        const int r = item - w.head * per_head;
        int lo = 0, hi = nseg;  // last segment whose prefix is <= r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (seg_prefix[mid] <= r) lo = mid;
            else hi = mid;
        }
        seg = lo;
        bx = r - seg_prefix[seg];
    } else {
        bx = item % nblk_x;
        const int rest = item / nblk_x;
        seg = rest % nseg;
        w.head = rest / nseg;
    }
    w.s0 = cu ? cu[seg] : 0;
    w.s1 = cu ? cu[seg + 1] : kv_total;
    const int seg_len = w.s1 - w.s0;
    // Query rows of this launch: global rows [q_begin, q_end) (the whole packed sequence for plain self-attention; a
    // slice when the query rows are sharded).  q / out / lse are indexed by (global row - q_begin); k / v by global row.
    const int q_lo = q_free ? q_begin : max(w.s0, q_begin);
    w.q_hi = q_free ? q_end : min(w.s1, q_end);
    w.q_row0 = q_lo + bx * (kTiles * kBlockM);
    w.valid = w.q_row0 < w.q_hi;
    w.n_mt = min(kTiles, (w.q_hi - w.q_row0 + kBlockM - 1) / kBlockM);  // query tiles with at least one valid row
    w.n_kv = (seg_len + kBlockN - 1) / kBlockN;
    w.ragged_tail = (seg_len % kBlockN) != 0;
    if (k_parts > 1) {
        const int per_part = (w.n_kv + k_parts - 1) / k_parts;
        const int t0 = w.kpart * per_part, t1 = min(w.n_kv, t0 + per_part);
        if (t0 >= t1) {
            w.valid = false;
        } else {
            const int s0 = w.s0;
            w.s0 = s0 + t0 * kBlockN;
            w.s1 = min(w.s1, s0 + t1 * kBlockN);
            w.n_kv = t1 - t0;
            w.ragged_tail = ((w.s1 - w.s0) % kBlockN) != 0;
        }
    }
    return w;
}

// Persistent kernel: one CTA per SM walks the work items item = blockIdx.x, blockIdx.x + gridDim.x, ...  Every role
// runs the same item loop on its own; the barriers' phases simply keep counting across items, so the producer
// streams the next item's K/V (and, once the last Q K^T of the current item has completed, its Q) while the softmax
// groups are still finishing the current one.
// kPrefix selects the work list at compile time, so that launches with few segments carry none of the table's code.
template <bool kBF16, bool kPrefix>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const void *__restrict__ bias_ptr,
                      const int *__restrict__ cu, float scale_log2, float inv_scale, void *__restrict__ out_ptr, int64_t o_rs,
                      float *__restrict__ lse, int q_begin, int q_end, int nblk_x, int nseg, int num_heads,
                      const int *__restrict__ max_len_dev, unsigned int *__restrict__ status, int kv_total, int q_free_flag,
                      int k_parts, long long part_o, long long part_l) {
    using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
    extern __shared__ uint8_t smem_raw[];
    SharedStorage &sh = *reinterpret_cast<SharedStorage *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    // The host sizes the work list from an upper bound of the longest segment.  A caller that cannot read the true
    // length back (a captured graph serving every merge mask) passes a loose bound plus the true one in device memory:
    // the work list then shrinks to the query blocks that can exist, and the round-robin over CTAs stays balanced.
    if (max_len_dev != nullptr) {
        const int m = min(max(*max_len_dev, 0), q_end - q_begin);
        nblk_x = min(nblk_x, (m + kTiles * kBlockM - 1) / (kTiles * kBlockM));
    }
    // Work list.  Launches with many segments (kMinPrefixSegs .. kMaxPrefixSegs): every CTA scans the segments' query-block
    // counts into shared memory and the items are exactly the blocks that exist.  With ragged segments a list with one
    // slot per (segment, maximal block index) unbalances the round-robin: the empty slots all carry the same block index,
    // and 148 CTAs is a multiple of 4 blocks per segment (0.81 balance on 64 ragged segments, 0.95 without the empty
    // slots).  Launches with few segments keep the slot list: the scan would cost them ~1.5 us for nothing.
    constexpr bool use_prefix = kPrefix;  // the host instantiates and sizes the shared memory by the segment count
    int *prefix_table = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(&sh) + sizeof(SharedStorage));
    if constexpr (kPrefix) {
        constexpr int kPer = kMaxPrefixSegs / kThreads;  // consecutive segments per thread
        int local[kPer], sum = 0;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int sg = threadIdx.x * kPer + i;
            local[i] = sg < nseg ? segment_blocks(sg, cu, q_begin, q_end) : 0;
            sum += local[i];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, d);
            if ((threadIdx.x & 31) >= d) incl += v;
        }
        if ((threadIdx.x & 31) == 31) sh.scan_warp[threadIdx.x >> 5] = incl;
        __syncthreads();
        int before = incl - sum;
        for (int wq = 0; wq < (int)(threadIdx.x >> 5); ++wq) before += sh.scan_warp[wq];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int sg = threadIdx.x * kPer + i;
            if (sg <= nseg) prefix_table[sg] = before;
            before += local[i];
        }
        if (nseg == kMaxPrefixSegs && threadIdx.x == kThreads - 1) prefix_table[kMaxPrefixSegs] = before;  // the grand total
        __syncthreads();
    }
    const int *seg_prefix = use_prefix ? prefix_table : nullptr;
    const int total_items = (use_prefix ? prefix_table[nseg] * num_heads : nblk_x * nseg * num_heads) * k_parts;
    const bool has_bias = bias_ptr != nullptr;
    const bool q_free = q_free_flag != 0;
    // a key tile needs the bias step when there is a bias, or when it is the partial last tile (masking)
    auto uses_slab = [&](const WorkItem &w, int j) { return has_bias || (w.ragged_tail && j == w.n_kv - 1); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        // an earlier CTA that gave up leaves the status word raised: later CTAs then skip their work
        sh.abort_flag = (*(volatile unsigned int *)status != 0) ? 1u : 0u;
        for (int i = 0; i < kTiles; ++i) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&sh.q_full[i][b], 1);
                mbar_init(&sh.q_empty[i][b], 1);
            }
            mbar_init(&sh.s_full[i], 1);
            mbar_init(&sh.p_full[i], kBlockM);
            mbar_init(&sh.o_done[i], 1);
            mbar_init(&sh.s_empty[i], kBlockM);
        }
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sh.kv_full[i], 1);
            mbar_init(&sh.kv_empty[i], kTiles);  // released by every issuer warp (an idle one arrives without an MMA)
        }
        for (int i = 0; i < kSlabStages; ++i) {
            mbar_init(&sh.slab_full[i], 1);
            mbar_init(&sh.slab_empty[i], kTiles);
        }
        mbar_init(&sh.q_slab_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kIssuerWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    // Register budget: the producer / issuer warpgroup needs few registers and hands its share to the three softmax
    // warpgroups (12 x 32 x 152 + 4 x 32 x 56 = 65536).  Each role branch below starts with its setmaxnreg; every warp
    // of a warpgroup has to execute it.
    const bool dead = sh.abort_flag != 0;  // read after the barrier: uniform for the CTA

    if (dead) {
        // fall through to the common exit
    } else if (warp == kProducerWarp) {
        // ===== producer =====================================================================================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        const T *bias = reinterpret_cast<const T *>(bias_ptr);
        bool ok = true;
        {   // the constant A side of the bias step: columns 0 and 1 are 1.0.  Both slabs are bfloat16 whatever the
            // q/k/v dtype (the bias step is an MMA instruction of its own): bias/scale and the mask value need its range.
            const uint32_t ones = pack2<true>(1.0f, 1.0f);
            const uint32_t qs = smem_u32(sh.q_slab);
#pragma unroll
            for (int i = 0; i < 4; ++i) slab_write_row(qs, lane * 4 + i, ones);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.q_slab_full);
        }
        int it = 0;            // K/V ring position, advanced once per K or V tile in the order K0 V0 K1 V1 ...
        int slab_it = 0;       // bias slab ring position, advanced once per key tile that uses the bias step
        int q_uses[kTiles] = {};  // items that loaded query tile t so far (buffer and phase of q_full / q_empty)
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const WorkItem w = decode_item<kPrefix>(item, nblk_x, nseg, cu, q_begin, q_end, seg_prefix, kv_total, q_free, k_parts);
            if (!w.valid) continue;
            if (lane == 0) {
                for (int t = 0; t < w.n_mt && ok; ++t) {
                    // Use n of query tile t goes to buffer n & 1, which is free once the last Q K^T of use n - 2 has completed:
                    // the query tiles of the next item are in flight while the current item is still being computed.
                    const int n = q_uses[t], b = n & 1;
                    if (n >= 2) ok = mbar_wait(&sh.q_empty[t][b], ((n >> 1) - 1) & 1, sh, status, kErrQFull);
                    if (ok) {
                        mbar_arrive_expect_tx(&sh.q_full[t][b], kQTileBytes);
                        tma_load_3d(sh.q[t][b], &map_q, 0, w.head, w.q_row0 - q_begin + t * kBlockM, &sh.q_full[t][b]);
                    }
                }
            }
            for (int t = 0; t < w.n_mt; ++t) ++q_uses[t];
            ok = __all_sync(0xffffffffu, ok);
            for (int j = 0; j < w.n_kv && ok; ++j) {
                if (uses_slab(w, j)) {
                    const int bs = slab_it % kSlabStages;
                    ok = mbar_wait(&sh.slab_empty[bs], ((slab_it / kSlabStages) & 1) ^ 1, sh, status, kErrSlabEmpty);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const uint32_t ks = smem_u32(sh.k_slab[bs]);
#pragma unroll
                    for (int i = 0; i < kBlockN / 32; ++i) {
                        const int r = lane * (kBlockN / 32) + i;
                        const int key = w.s0 + j * kBlockN + r;
                        float hi = kMasked, lo = 0.0f;
                        if (key < w.s1) {
                            const float b = has_bias ? Elem<T>::to_f32(bias[key]) * inv_scale : 0.0f;
                            hi = __bfloat162float(__float2bfloat16_rn(b));
                            lo = b - hi;
                        }
                        slab_write_row(ks, r, pack2<true>(hi, lo));
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.slab_full[bs]);
                    ++slab_it;
                }
                if (lane == 0) {
#pragma unroll
                    for (int kv = 0; kv < 2 && ok; ++kv) {  // K tile, then V tile of the same keys
                        const int stage = (it + kv) % kStages;
                        ok = mbar_wait(&sh.kv_empty[stage], (((it + kv) / kStages) & 1) ^ 1, sh, status, kErrKvEmpty);
                        if (ok) {
                            mbar_arrive_expect_tx(&sh.kv_full[stage], kKvTileBytes);
                            tma_load_3d(sh.kv[stage], kv == 0 ? &map_k : &map_v, 0, w.head, w.s0 + j * kBlockN, &sh.kv_full[stage]);
                        }
                    }
                }
                ok = __all_sync(0xffffffffu, ok);
                it += 2;
            }
        }
    } else if (warp >= kIssuerWarp0) {
        // ===== MMA issuer of query tile t (all lanes run the loop, one elected lane issues) ================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        const int t = warp - kIssuerWarp0;
        constexpr uint32_t idesc_qk = make_idesc(kBF16, kBlockM, kBlockN, false);
        constexpr uint32_t idesc_slab = make_idesc(true, kBlockM, kBlockN, false);
        constexpr uint32_t idesc_pv = make_idesc(kBF16, kBlockM, kHeadDim, true);
        const uint64_t q_desc0 = make_smem_desc(smem_u32(sh.q[t][0]));  // buffer b: + b * (kQTileBytes >> 4)
        const uint64_t q_slab_desc = make_smem_desc(smem_u32(sh.q_slab));
        const uint64_t kv_desc0 = make_smem_desc(smem_u32(sh.kv[0]));       // slot i: + i * (kKvTileBytes >> 4)
        const uint64_t k_slab_desc0 = make_smem_desc(smem_u32(sh.k_slab[0]));
        const uint32_t s_tmem = tmem + kTmemS + t * kBlockN;
        const uint32_t o_tmem = tmem + kTmemO + t * kHeadDim;
        const uint32_t p_tmem = tmem + kTmemP + t * (kBlockN / 2);
        bool ok = mbar_wait(&sh.q_slab_full, 0, sh, status, kErrQFull);
        ok = __all_sync(0xffffffffu, ok);
        int it = 0;        // K/V ring position at the start of the current item (same count as the producer's)
        int slab_it = 0;   // bias slab ring position
        int step = 0;      // key tiles this query tile has processed so far (phase of s_full / s_empty / p_full / o_done)
        int q_uses = 0;    // items in which this query tile was active (phase of q_full / q_empty)
        TRACE_DECL();
#ifdef COME_ATTN_TRACE
        const long long tr_start = clock64();
#endif
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const WorkItem w = decode_item<kPrefix>(item, nblk_x, nseg, cu, q_begin, q_end, seg_prefix, kv_total, q_free, k_parts);
            if (!w.valid) continue;
            if (t >= w.n_mt) {
                // This query tile is empty in this item: release the K/V and slab slots without using them, so that the
                // rings' arrival counts do not depend on the item.
                for (int j = 0; j < w.n_kv && ok; ++j) {
#pragma unroll
                    for (int kv = 0; kv < 2 && ok; ++kv) {
                        const int x = it + 2 * j + kv, slot = x % kStages;
                        ok = mbar_wait(&sh.kv_full[slot], (x / kStages) & 1, sh, status, kErrKvFull);
                        ok = __all_sync(0xffffffffu, ok);
                        if (ok && lane == 0) mbar_arrive(&sh.kv_empty[slot]);
                    }
                    if (ok && uses_slab(w, j)) {
                        const int bs = slab_it % kSlabStages;
                        ok = mbar_wait(&sh.slab_full[bs], (slab_it / kSlabStages) & 1, sh, status, kErrSlabFull);
                        ok = __all_sync(0xffffffffu, ok);
                        if (ok && lane == 0) mbar_arrive(&sh.slab_empty[bs]);
                        ++slab_it;
                    }
                }
                it += 2 * w.n_kv;
                continue;
            }
            const int qb = q_uses & 1;
            ok = mbar_wait(&sh.q_full[t][qb], (q_uses >> 1) & 1, sh, status, kErrQFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint64_t q_desc = q_desc0 + (uint64_t)(qb * (kQTileBytes >> 4));
            // S(0), then per key tile j: S(j+1) = Q K_(j+1)^T as soon as the softmax group has read S(j) into registers,
            // and O += P(j) V_j as soon as P(j) is staged.  Ring slot of K_j is 2j, of V_j is 2j+1 (from `it`).  The other
            // query tile's issuer runs the same loop independently.
            // S(jj) = Q K_jj^T (+ the bias step): what it waits for, and its instructions
            auto wait_s = [&](int jj) -> bool {
                const int k_it = it + 2 * jj, k_slot = k_it % kStages;
                const int bs = slab_it % kSlabStages;
                TRACE_BEGIN();
                bool good = mbar_wait(&sh.kv_full[k_slot], (k_it / kStages) & 1, sh, status, kErrKvFull);
                if (good && uses_slab(w, jj)) good = mbar_wait(&sh.slab_full[bs], (slab_it / kSlabStages) & 1, sh, status, kErrSlabFull);
                TRACE_END(0);
                TRACE_BEGIN();
                // the softmax group must have pulled the previous scores (also those of the previous item) out of S
                if (good && step + jj > 0) good = mbar_wait(&sh.s_empty[t], (step + jj - 1) & 1, sh, status, kErrSEmpty);
                TRACE_END(1);
                TRACE_STAMP(8, step + jj == 65);
                return __all_sync(0xffffffffu, good);
            };
            auto emit_s = [&](int jj) {
                const int k_it = it + 2 * jj, k_slot = k_it % kStages;
                const bool slab = uses_slab(w, jj);
                const int bs = slab_it % kSlabStages;
                const uint64_t k_desc = kv_desc0 + (uint64_t)(k_slot * (kKvTileBytes >> 4));
                if (elect_one()) {  // one lane issues the whole group: a single election and branch instead of one per instruction
                    tc_mma_ss_1(s_tmem, q_desc + 0, k_desc + 0, idesc_qk, 0u);
                    tc_mma_ss_1(s_tmem, q_desc + 2, k_desc + 2, idesc_qk, 1u);
                    tc_mma_ss_1(s_tmem, q_desc + 4, k_desc + 4, idesc_qk, 1u);
                    tc_mma_ss_1(s_tmem, q_desc + 6, k_desc + 6, idesc_qk, 1u);
                    if (slab) tc_mma_ss_1(s_tmem, q_slab_desc, k_slab_desc0 + (uint64_t)(bs * (kKvTileBytes >> 4)), idesc_slab, 1u);
                    tc_commit_1(&sh.s_full[t]);
                    tc_commit_1(&sh.kv_empty[k_slot]);
                    if (slab) tc_commit_1(&sh.slab_empty[bs]);
                    if (jj == w.n_kv - 1) tc_commit_1(&sh.q_empty[t][qb]);
                }
                __syncwarp();
                if (slab) ++slab_it;
                TRACE_STAMP(11, step + jj == 65);
            };
            // O += P(j) V_j: what it waits for, and its instructions
            auto wait_pv = [&](int j) -> bool {
                const int v_it = it + 2 * j + 1, v_slot = v_it % kStages;
                TRACE_BEGIN();
                bool good = mbar_wait(&sh.kv_full[v_slot], (v_it / kStages) & 1, sh, status, kErrKvFull);
                TRACE_END(2);
                TRACE_BEGIN();
                if (good) good = mbar_wait(&sh.p_full[t], (step + j) & 1, sh, status, kErrPFull);
                TRACE_END(3);
                TRACE_COUNT(5, 1);
                TRACE_STAMP(9, step + j == 64);
                return __all_sync(0xffffffffu, good);
            };
            auto emit_pv = [&](int j) {
                const int v_it = it + 2 * j + 1, v_slot = v_it % kStages;
                const uint64_t v_desc = kv_desc0 + (uint64_t)(v_slot * (kKvTileBytes >> 4));
                // 16 keys per instruction: 8 columns of 16-bit pairs of P, 16 rows (2048 bytes) of the V tile
                if (elect_one()) {
#pragma unroll
                    for (int i = 0; i < kBlockN / 16; ++i)
                        tc_mma_ts_1(o_tmem, p_tmem + 8 * i, v_desc + (uint64_t)(i * 128), idesc_pv, (j > 0 || i > 0) ? 1u : 0u);
                    tc_commit_1(&sh.o_done[t]);
                    tc_commit_1(&sh.kv_empty[v_slot]);
                }
                __syncwarp();
                TRACE_STAMP(10, step + j == 64);
            };
            ok = wait_s(0);
            if (ok) {
                tc_fence_after();
                emit_s(0);
            }
            for (int j = 0; j < w.n_kv && ok; ++j) {
                if (j + 1 < w.n_kv) {
                    ok = wait_s(j + 1);
                    if (!ok) break;
                    tc_fence_after();
                    emit_s(j + 1);
                }
                ok = wait_pv(j);
                if (!ok) break;
                tc_fence_after();
                emit_pv(j);
            }
            it += 2 * w.n_kv;
            step += w.n_kv;
            ++q_uses;
        }
#ifdef COME_ATTN_TRACE
        tr_acc[4] = clock64() - tr_start;
#endif
        TRACE_FLUSH();
        __syncwarp();
    } else {
        // ===== softmax group of query tile t ================================================================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
        const int t = warp >> 2;
        const int r = threadIdx.x & 127;                          // row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem + lane_addr + kTmemS + t * kBlockN;
        const uint32_t o_tmem = tmem + lane_addr + kTmemO + t * kHeadDim;
        const uint32_t p_tmem = tmem + lane_addr + kTmemP + t * (kBlockN / 2);
        bool ok = true;
        int step = 0;  // key tiles processed so far by this query tile: phase of s_full / s_empty / p_full / o_done
        TRACE_DECL();
#ifdef COME_ATTN_TRACE
        const long long tr_start = clock64();
#endif
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const WorkItem w = decode_item<kPrefix>(item, nblk_x, nseg, cu, q_begin, q_end, seg_prefix, kv_total, q_free, k_parts);
            if (!w.valid || t >= w.n_mt) continue;
            const int n_kv = w.n_kv;
            const int row = w.q_row0 + t * kBlockM + r;
            float m_ref = -INFINITY, l = 0.0f;  // reference max (log2 units, scale applied) and running sum

            for (int j = 0; j < n_kv && ok; ++j) {
                TRACE_BEGIN();
                ok = mbar_wait(&sh.s_full[t], (step + j) & 1, sh, status, kErrSFull);
                TRACE_END(0);
                TRACE_COUNT(5, 1);
                TRACE_STAMP(8, step + j == 64);
                TRACE_STAMP(9, step + j == 65);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                TRACE_BEGIN();
                // The whole row of kBlockN scores is pulled into registers at once, which frees S for the next Q K^T right
                // away; the row is then turned into probabilities 32 columns at a time.
                constexpr int kQuarters = kBlockN / 32;
                uint32_t srow[kQuarters][32];
#pragma unroll
                for (int q = 0; q < kQuarters; ++q) tmem_ld32(s_tmem + 32 * q, srow[q]);
                tc_wait_ld();
                TRACE_END(1);
                tc_fence_before();
                mbar_arrive(&sh.s_empty[t]);
                bool o_ready = (j == 0);  // P V of the previous key tile complete: O stable, P buffer free
                // Row max over all scores first: independent 3-input chains of 16 scores keep the ALU pipe fed, and the
                // rare rescale is decided once per key tile, so the exponentials below are one straight-line block.
                float t_max = -INFINITY;
#pragma unroll
                for (int c = 0; c < 2 * kQuarters; ++c) {
                    const uint32_t *e = &srow[c >> 1][(c & 1) * 16];
                    float m = max3(__uint_as_float(e[0]), __uint_as_float(e[1]), __uint_as_float(e[2]));
#pragma unroll
                    for (int i = 3; i < 15; i += 2) m = max3(m, __uint_as_float(e[i]), __uint_as_float(e[i + 1]));
                    t_max = max3(t_max, m, __uint_as_float(e[15]));
                }
                t_max *= scale_log2;
                const bool need = t_max > m_ref + kRescaleThreshold;  // always true on the first key tile (m_ref = -inf)
                if (__any_sync(0xffffffffu, need)) {
                    float alpha = 1.0f;
                    if (need) {
                        alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - t_max);
                        m_ref = t_max;
                        l *= alpha;
                    }
                    if (j > 0) {  // rescale what earlier key tiles accumulated
                        ok = mbar_wait(&sh.o_done[t], (step + j - 1) & 1, sh, status, kErrODone);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        o_ready = true;
                        scale_accumulator(o_tmem, alpha);
                    }
                }
                // p = 2^(s * scale*log2e - m_ref), two scores per instruction; a share of the pairs takes the polynomial
                // route so that the special-function unit and the FMA pipe split the exponentials.
                const f32x2_t scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(-m_ref, -m_ref);
                f32x2_t sum2 = pack_f32x2(0.0f, 0.0f);
                auto quarter = [&](const uint32_t(&a)[32], uint32_t(&pk)[16]) {
#pragma unroll
                    for (int pair = 0; pair < 16; ++pair) {
                        const f32x2_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(a[2 * pair]), __uint_as_float(a[2 * pair + 1])), scale2, neg_m2);
                        float x0, x1, p0, p1;
                        unpack_f32x2(x2, x0, x1);
                        if ((kPolyPairs >> pair) & 1u) {
                            exp2_poly_x2(x0, x1, p0, p1);
                        } else {
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        sum2 = add_f32x2(sum2, pack_f32x2(p0, p1));
                        pk[pair] = pack2<kBF16>(p0, p1);
                    }
                };
                {
                    uint32_t pk[16];
                    quarter(srow[0], pk);
                    if (!o_ready) {  // the P buffer is free once P V of the previous key tile has completed
                        TRACE_BEGIN();
                        ok = mbar_wait(&sh.o_done[t], (step + j - 1) & 1, sh, status, kErrODone);
                        TRACE_END(2);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    tmem_st16(p_tmem, pk);  // 32 keys -> 16 columns of 16-bit pairs
                }
#pragma unroll
                for (int q = 1; q < kQuarters; ++q) {
                    uint32_t pk[16];
                    quarter(srow[q], pk);
                    tmem_st16(p_tmem + 16 * q, pk);
                }
                {
                    float s_lo, s_hi;
                    unpack_f32x2(sum2, s_lo, s_hi);
                    l += s_lo + s_hi;
                }
                if (!ok) break;
                TRACE_BEGIN();
                tc_wait_st();
                TRACE_END(3);
                tc_fence_before();
                mbar_arrive(&sh.p_full[t]);
                TRACE_STAMP(10, step + j == 64);
            }

            TRACE_BEGIN();
            if (ok) {
                ok = mbar_wait(&sh.o_done[t], (step + n_kv - 1) & 1, sh, status, kErrODone);
                ok = __all_sync(0xffffffffu, ok);
            }
            TRACE_END(6);
            TRACE_BEGIN();
            if (ok) {
                tc_fence_after();
                uint32_t o[2][32];
                tmem_ld32(o_tmem + 0, o[0]);
                tmem_ld32(o_tmem + 32, o[1]);
                tc_wait_ld();  // O is in registers: the next item's first P V may overwrite the accumulator
                if (row < w.q_hi) {
                    const float inv = 1.0f / l;
                    // The row's 64 outputs as 32 packed words, written with 32-byte stores where the address allows it:
                    // a warp's store then covers whole 32-byte sectors of its 32 rows instead of halves.
                    uint32_t pk[32];
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            pk[c * 16 + i / 2] = pack2<kBF16>(__uint_as_float(o[c][i]) * inv, __uint_as_float(o[c][i + 1]) * inv);
                    T *dst_row = reinterpret_cast<T *>(out_ptr) + (int64_t)w.kpart * part_o + (int64_t)(row - q_begin) * o_rs + (int64_t)w.head * kHeadDim;
                    if ((reinterpret_cast<uintptr_t>(dst_row) & 31) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst_row + 2 * i),
                                         "r"(pk[i]), "r"(pk[i + 1]), "r"(pk[i + 2]), "r"(pk[i + 3]), "r"(pk[i + 4]), "r"(pk[i + 5]),
                                         "r"(pk[i + 6]), "r"(pk[i + 7])
                                         : "memory");
                    } else {
                        uint4 *dst = reinterpret_cast<uint4 *>(dst_row);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) dst[i / 4] = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
                    }
                    if (lse) lse[(int64_t)w.kpart * part_l + (int64_t)w.head * (q_end - q_begin) + (row - q_begin)] = (m_ref + log2f(l)) * kLn2;
                }
            }
            TRACE_END(7);
            step += n_kv;
        }
#ifdef COME_ATTN_TRACE
        tr_acc[4] = clock64() - tr_start;
#endif
        TRACE_FLUSH();
    }

    // ===== common exit ==========================================================================================
    tc_fence_before();
    __syncthreads();
    if (sh.abort_flag != 0) {
        // give loads that may still be in flight time to land before the shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (warp == kIssuerWarp0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Self-test of the failure path: one CTA waits, with the attention kernel's own bounded wait, on a barrier that nothing
// ever arrives at.  The wait gives up after `ticks` clocks, raises the CTA's abort flag and the device status word, and
// the kernel returns normally; `waited_out` (optional) receives the clocks it waited.
__global__ void selftest_wait_kernel(long long ticks, unsigned int *__restrict__ status, long long *__restrict__ waited_out) {
    __shared__ alignas(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long t0 = clock64();
    const bool ok = mbar_wait_limit(&bar, 0, &abort_flag, status, kErrSelfTest, ticks);
    if (threadIdx.x == 0 && waited_out) *waited_out = ok ? -1 : clock64() - t0;
}

// ---- host side --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// [total, H, 64] view with arbitrary row stride; box = box_rows rows x 1 head x 64 elements, 128-byte swizzle.
// A tensor map is a pure function of these arguments (it holds an address, not a snapshot of memory), so each host
// thread keeps the last few it encoded: a model that calls attention layer after layer on the same buffers encodes
// them once instead of three times per launch.
struct MapKey {
    const void *base;
    int64_t total, row_stride;
    int dtype, H, box_rows;
    bool operator==(const MapKey &o) const {
        return base == o.base && total == o.total && row_stride == o.row_stride && dtype == o.dtype && H == o.H && box_rows == o.box_rows;
    }
};
constexpr int kMapCacheSlots = 16;
struct MapCache {
    MapKey key[kMapCacheSlots];
    CUtensorMap map[kMapCacheSlots];
    bool used[kMapCacheSlots];
    int next;
};

int make_map(CUtensorMap *map, const void *base, int dtype, int64_t total, int H, int64_t row_stride, int box_rows) {
    thread_local MapCache cache = {};
    const MapKey key{base, total, row_stride, dtype, H, box_rows};
    for (int i = 0; i < kMapCacheSlots; ++i)
        if (cache.used[i] && cache.key[i] == key) {
            *map = cache.map[i];
            return COME_OK;
        }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
        return COME_ERR_CUDA;
    }
    cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)H, (cuuint64_t)total};
    cuuint64_t strides[2] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)row_stride * 2};
    cuuint32_t box[3] = {(cuuint32_t)kHeadDim, 1, (cuuint32_t)box_rows};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dtype == COME_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return COME_ERR_CUDA;
    }
    const int slot = cache.next;
    cache.next = (slot + 1) % kMapCacheSlots;
    cache.key[slot] = key;
    cache.map[slot] = *map;
    cache.used[slot] = true;
    return COME_OK;
}

}  // namespace

bool attn_sm100_supported(const AttnArgs &a) {
    if (a.D != kHeadDim) return false;
    if (a.dtype != COME_BF16 && a.dtype != COME_F16) return false;
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    if (!al16(a.q) || !al16(a.k) || !al16(a.v) || !al16(a.out)) return false;
    if (a.q_rs % 8 || a.k_rs % 8 || a.v_rs % 8 || a.o_rs % 8) return false;
    // the row max is taken on raw scores and the bias is divided by the scale: both need a positive finite scale
    if (!(a.scale > 0.0f) || !(a.scale < 3.0e38f)) return false;
    return true;
}

// The shared-memory opt-in of a kernel is set once per device and instantiation (not again on every launch, so that
// launches stay cheap and legal inside a stream capture).  Host threads may race to the first launch: the flag is
// raised only after cudaFuncSetAttribute has succeeded, under a mutex, so no thread launches before the opt-in exists
// and a failed attempt is retried by the next launch.
template <typename Kernel> static int ensure_smem_optin(Kernel kernel, int slot, size_t smem) {
    static std::mutex mu;
    static bool done[64][4];
    int dev = 0;
    COME_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("come_attn_varlen_fwd: device ordinal %d is out of the supported range", dev);
        return COME_ERR_ARG;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev][slot]) return COME_OK;
    COME_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    done[dev][slot] = true;
    return COME_OK;
}

// Upper bound on the CTAs of the persistent kernel for launches issued by this host thread (0 = one per SM).
static thread_local int t_cta_limit = 0;
void attn_sm100_set_cta_limit(int max_ctas) { t_cta_limit = max_ctas > 0 ? max_ctas : 0; }

int attn_sm100_launch(const AttnArgs &a, cudaStream_t stream) {
    unsigned int *status = status_word_dev();
    if (!status) return COME_ERR_CUDA;
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map(&mq, a.q, a.dtype, a.q_end - a.q_begin, a.H, a.q_rs, kBlockM)) != COME_OK) return rc;
    if ((rc = make_map(&mk, a.k, a.dtype, a.total, a.H, a.k_rs, kBlockN)) != COME_OK) return rc;
    if ((rc = make_map(&mv, a.v, a.dtype, a.total, a.H, a.v_rs, kBlockN)) != COME_OK) return rc;
    const bool with_table = !a.q_free && a.nseg >= kMinPrefixSegs && a.nseg <= kMaxPrefixSegs;
    const size_t smem = sizeof(SharedStorage) + 1024 + (with_table ? kPrefixTableBytes : 0);
    const int64_t q_rows = a.q_end - a.q_begin;
    const int64_t span = a.q_free ? q_rows : (a.max_seqlen < q_rows ? a.max_seqlen : q_rows);  // most query rows any segment can own here
    const int nblk_x = (int)((span + kTiles * kBlockM - 1) / (kTiles * kBlockM));
    const int k_parts = a.k_parts > 1 ? a.k_parts : 1;
    if (k_parts > 1) {
        // shares of the key tiles of every item: one segment whose keys all query rows attend to; no share may be empty
        const int64_t tiles = (a.total + kBlockN - 1) / kBlockN, per_part = (tiles + k_parts - 1) / k_parts;
        if (!a.q_free || a.lse == nullptr || (int64_t)(k_parts - 1) * per_part >= tiles) {
            set_error("attention with %d key shares needs the one-segment cross form, a log-sum-exp output and at least one "
                      "key tile per share (%lld tiles)", k_parts, (long long)tiles);
            return COME_ERR_ARG;
        }
    }
    const int64_t items = (int64_t)nblk_x * a.nseg * a.H * k_parts;
    if (items <= 0) return COME_OK;
    if (items >= (1ll << 31)) {
        set_error("come_attn_varlen_fwd: %lld work items do not fit 32 bits", (long long)items);
        return COME_ERR_ARG;
    }
    int sms = sm_count();
    if (t_cta_limit > 0 && t_cta_limit < sms) sms = t_cta_limit;
    const unsigned grid = (unsigned)(items < sms ? items : sms);  // persistent: one CTA per SM walks the items
    const float scale_log2 = a.scale * kLog2e;
    const float inv_scale = 1.0f / a.scale;
#define COME_ATTN_LAUNCH(BF16, PREFIX, SLOT)                                                                                   \
    do {                                                                                                                       \
        if ((rc = ensure_smem_optin(attn_fwd_sm100_kernel<BF16, PREFIX>, SLOT, smem)) != COME_OK) return rc;                    \
        attn_fwd_sm100_kernel<BF16, PREFIX><<<grid, kThreads, smem, stream>>>(mq, mk, mv, a.bias, a.cu, scale_log2, inv_scale, a.out, \
                                                                              a.o_rs, a.lse, (int)a.q_begin, (int)a.q_end, nblk_x,   \
                                                                              a.nseg, a.H, a.max_seqlen_dev, status, (int)a.total,   \
                                                                              a.q_free ? 1 : 0, k_parts, (long long)a.part_o,        \
                                                                              (long long)a.part_l);                                  \
    } while (0)
    if (a.dtype == COME_BF16) {
        if (with_table) COME_ATTN_LAUNCH(true, true, 0);
        else COME_ATTN_LAUNCH(true, false, 1);
    } else {
        if (with_table) COME_ATTN_LAUNCH(false, true, 2);
        else COME_ATTN_LAUNCH(false, false, 3);
    }
#undef COME_ATTN_LAUNCH
    return check_launch("come_attn_varlen_fwd (tcgen05 kernel)");
}

}  // namespace come

extern "C" int come_selftest_bounded_wait(int64_t ticks, int64_t *waited_dev, void *stream) {
    COME_REQUIRE(ticks > 0 && ticks <= (1ll << 26), "come_selftest_bounded_wait: ticks must be in (0, 2^26] (a fraction of a second)");
    unsigned int *status = come::status_word_dev();
    if (!status) return COME_ERR_CUDA;
    come::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)ticks, status, (long long *)waited_dev);
    return come::check_launch("come_selftest_bounded_wait");
}

#ifdef COME_ATTN_TRACE
// Development builds only: copies the per-warp wait counters of the last attention launch to host memory.
extern "C" int come_debug_attn_trace(unsigned long long *host_out, int n_words) {
    const size_t bytes = sizeof(unsigned long long) * (size_t)n_words;
    if (bytes > sizeof(come::g_attn_trace)) return COME_ERR_ARG;
    return cudaMemcpyFromSymbol(host_out, come::g_attn_trace, bytes) == cudaSuccess ? COME_OK : COME_ERR_CUDA;
}
#endif
