// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (TMEM allocation, UMMA,
// UTCCP scale-factor copy, TMEM loads) and the shared-memory / instruction descriptors the tensor core reads.
//
// Every wait in this file is bounded: a barrier that does not flip within WAIT_LIMIT_CYCLES makes the waiter
// record an error code in a device status word, raise a CTA-wide abort flag and return false, so that a
// synchronisation bug ends the kernel with an error status instead of hanging the GPU.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace blaze {

// Device status codes written to the status word (0 = OK).  The host turns any non-zero value into
// ACLTENSOR_STATUS_EXECUTION_FAILED.
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_TIMEOUT_SMEM_FULL = 1,    // MMA warp waited for a TMA stage that never arrived
    DEV_TIMEOUT_SMEM_EMPTY = 2,   // TMA warp waited for a stage that was never released
    DEV_TIMEOUT_TMEM_FULL = 3,    // epilogue waited for an accumulator that never completed
    DEV_TIMEOUT_TMEM_EMPTY = 4,   // MMA warp waited for an accumulator that was never drained
    DEV_TIMEOUT_FIXUP_FLAG = 5,   // stream-K owner waited for a partial tile that was never published
    DEV_TIMEOUT_PEER = 6,         // 2-CTA pair: waited for the partner CTA
    DEV_TIMEOUT_SELFTEST = 7,     // the diagnostic kernel's wait on a barrier nobody signals (expected to expire)
};

#ifndef BLAZE_WAIT_LIMIT_CYCLES
#define BLAZE_WAIT_LIMIT_CYCLES (1LL << 30)      // about half a second at 2 GHz
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta_rank` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta_rank) {
    asm volatile(
        "{\n\t"
        ".reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t"
        "}\n" ::"r"(smem_u32(bar)),
        "r"(cta_rank)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Same, with cluster-scope acquire: needed when the arrival came from the partner CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory and is shared by every role of the CTA; `status` is the
// global status word.  Returns false when the wait was abandoned.
template <bool kClusterScope = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code, long long limit_cycles = BLAZE_WAIT_LIMIT_CYCLES) {
    auto probe = [&]() { return kClusterScope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (probe()) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (probe()) return true;
        }
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

// Lean forms for the single-thread issue loops, which pay for every instruction: barriers are named by their
// precomputed 32-bit shared-memory address.
__device__ __forceinline__ bool mbar_try_wait_addr(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
    if (mbar_try_wait_addr(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (mbar_try_wait_addr(bar, parity)) return true;
        }
        if (*abort_flag != 0) return false;
        if (clock64() - t0 > BLAZE_WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void mbar_arrive_expect_tx_addr(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void umma_commit_addr(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_2d_addr(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int x, int y,
                                                 uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "l"(hint)
        : "memory");
}

// ------------------------------------------------------------------------------------------------ global flags

// Flag hand-over between CTAs of one grid (stream-K partial tiles): release store / acquire load at GPU scope.
__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* ptr, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* ptr) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u64(unsigned long long* ptr, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(ptr), "l"(v) : "memory");
}

// ------------------------------------------------------------------------------------------------ dependent launch

// A kernel launched with programmatic stream serialisation may start while its predecessor in the stream is still
// running.  `grid_dependency_wait` blocks the calling thread until the predecessor grid has finished and its writes
// are visible; `grid_launch_dependents` lets the successor's blocks start being scheduled.  Both are no-ops for a
// plain launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ TMA

// L2 eviction-priority hints for TMA loads (opaque 64-bit policy words the hardware defines).
constexpr uint64_t kEvictNormal = 0x1000000000000000ull;
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load global -> shared, completing `bytes` on `bar`.  x is the innermost (contiguous) coordinate
// and must make x * element_size a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y,
                                            uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(hint)
        : "memory");
}

// Same load issued by either CTA of a 2-CTA pair: data lands in the issuing CTA's shared memory, the byte
// count is credited to the barrier at this offset in the pair's leader (even-ranked) CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x,
                                                 int y, uint64_t hint) {
    const uint32_t leader_bar = smem_u32(bar) & 0xFEFFFFFFu;
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(leader_bar), "r"(x), "r"(y), "l"(hint)
        : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Untiled bulk copy shared -> global (bulk-group completion); both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(gmem_dst)),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}

// 2-D tiled store shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
template <int kPending>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ------------------------------------------------------------------------------------------------ tcgen05 / TMEM

// All three allocation calls are warp-collective (.sync.aligned): call them with a full, converged warp.
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                     "r"(columns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                     "r"(columns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    }
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Make `bar` flip once every tcgen05.mma / tcgen05.cp this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 2-CTA form: arrives on the barrier at this offset in every CTA named by `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(cta_mask)
        : "memory");
}

__device__ __forceinline__ void umma_commit_pair_addr(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// Shared-memory operand descriptor for a K-major tile stored with the 128-byte swizzle TMA produces:
// rows are 128 bytes apart, groups of 8 rows are 1024 bytes apart (stride byte offset), the tile base is
// 1024-byte aligned and k steps inside the 128-byte row are taken by advancing the start address.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                       // descriptor version of this architecture
    d |= static_cast<uint64_t>(2) << 61;                       // layout type: 128-byte swizzle
    return d;
}

// Descriptor of an un-swizzled block of 32 rows x 16 bytes (8-row core matrices 128 bytes apart): the source
// shape of the scale-factor copy into TMEM.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// Descriptor for a 128-row x 32-byte block copied by tcgen05.cp.128x256b: rows 16 bytes apart in groups of eight
// (128 bytes per group), the second 16-byte half of every row `half_stride` bytes after the first.
__device__ __forceinline__ uint64_t umma_desc_sf_wide(uint32_t smem_addr, uint32_t half_stride) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(half_stride >> 4) << 16;        // leading byte offset between the two 16-byte halves
    d |= static_cast<uint64_t>(128 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

enum UmmaFormat : uint32_t { FMT_E4M3 = 0, FMT_E5M2 = 1, FMT_E2M1 = 5 };
constexpr uint32_t FMT_MXF4_E2M1 = 1;     // E2M1 in the format numbering of kind::mxf4

// Instruction descriptor for kind::f8f6f4 (fp32 accumulate, both operands K-major).
__host__ __device__ constexpr uint32_t umma_idesc_f8(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
    return (1u << 4)            // accumulator format: f32
           | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor for kind::mxf8f6f4.block_scale with E8M0 scales; a_sf / b_sf select which of the four
// scale bytes held in one TMEM column the instruction uses.
__host__ __device__ constexpr uint32_t umma_idesc_mx(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                     uint32_t a_sf, uint32_t b_sf) {
    return (b_sf << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23)   // scale format: E8M0
           | ((m >> 4) << 24) | (a_sf << 29);
}

template <int kCtaGroup>
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    if constexpr (kCtaGroup == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Four K=32 steps of one 128-byte-swizzled K block with kind::f8f6f4: the operand descriptors are given as the low
// word of the first step (start address in 16-byte units plus the constant fields) and the shared high word; each
// further step starts 32 bytes (2 units) later.  The first instruction overwrites the accumulator.
__device__ __forceinline__ void umma_f8_kblock(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                               uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p0, p1;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 la, lb;\n\t"
        "setp.ne.b32 p0, 0, 0;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p0;\n\t"
        "add.u32 la, %1, 2;\n\t"
        "add.u32 lb, %2, 2;\n\t"
        "mov.b64 da, {la, %3};\n\t"
        "mov.b64 db, {lb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p1;\n\t"
        "add.u32 la, %1, 4;\n\t"
        "add.u32 lb, %2, 4;\n\t"
        "mov.b64 da, {la, %3};\n\t"
        "mov.b64 db, {lb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p1;\n\t"
        "add.u32 la, %1, 6;\n\t"
        "add.u32 lb, %2, 6;\n\t"
        "mov.b64 da, {la, %3};\n\t"
        "mov.b64 db, {lb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p1;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc)
        : "memory");
}

template <int kCtaGroup>
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    if constexpr (kCtaGroup == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
            : "memory");
    }
}

// FP4 x FP4 with one E8M0 scale per 32 K: dense 4-bit operands (two codes per byte in shared memory), K = 64 per
// instruction, i.e. two scale bytes of each operand per instruction (ids 0 or 2 pick the byte pair of the TMEM cell).
// Twice the rate of kind::mxf8f6f4.  2-CTA form only.
__device__ __forceinline__ void umma_mxf4_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// Copy one 32-row x 16-byte scale-factor block from shared memory into 4 TMEM columns, replicated into all
// four 32-lane quadrants.
template <int kCtaGroup>
__device__ __forceinline__ void utccp_sf(uint32_t tmem_dst, uint64_t sf_desc) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sf_desc) : "memory");
    } else {
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sf_desc) : "memory");
    }
}

// Copy a 128-row x 32-byte block from shared memory into 8 TMEM columns of all 128 lanes (no broadcast).
template <int kCtaGroup>
__device__ __forceinline__ void utccp_sf_wide(uint32_t tmem_dst, uint64_t desc) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(tmem_dst), "l"(desc) : "memory");
    } else {
        asm volatile("tcgen05.cp.cta_group::2.128x256b [%0], %1;" ::"r"(tmem_dst), "l"(desc) : "memory");
    }
}

// Load 32 consecutive fp32 accumulator columns of this thread's TMEM lane (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
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
// Same for 64 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
          "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
          "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
          "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
          "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ cluster

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
    cluster_arrive();
    cluster_wait();
}

// ------------------------------------------------------------------------------------------------ epilogue math

enum Activation : int { ACT_IDENTITY = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_SIGMOID = 4, ACT_TANH = 5 };

// GELU, tanh form: 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3).  Since 0.5 (1 + tanh(u)) = 1 / (1 + e^(-2u)),
// it is evaluated as x / (1 + 2^w) with w = -2 u log2(e): one ex2 and one reciprocal, relative error ~1e-6, and the
// tails are exact limits (x -> +inf gives x, x -> -inf gives -0).
__device__ __forceinline__ float gelu_tanh_f32(float x) {
    const float k0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
    const float k1 = k0 * 0.044715f;
    const float w = x * fmaf(x * x, k1, k0);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(w));
    return __fdividef(x, 1.0f + e);
}

// 1 / (1 + 2^(-x log2 e)): one ex2 and one reciprocal; exact limits 0 and 1 at the tails.
__device__ __forceinline__ float sigmoid_f32(float x) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    return __fdividef(1.0f, 1.0f + e);
}

template <int kAct>
__device__ __forceinline__ float apply_act(float x) {
    if constexpr (kAct == ACT_RELU) return fmaxf(x, 0.0f);
    if constexpr (kAct == ACT_GELU_TANH) return gelu_tanh_f32(x);
    if constexpr (kAct == ACT_SILU) return x * sigmoid_f32(x);
    if constexpr (kAct == ACT_SIGMOID) return sigmoid_f32(x);
    if constexpr (kAct == ACT_TANH) return fmaf(2.0f, sigmoid_f32(2.0f * x), -1.0f);
    return x;
}

// (a0, a1) += (v0, v1) * s with one packed float32x2 FMA (two IEEE fused multiply-adds, same bits as two fmaf).
__device__ __forceinline__ void fma_f32x2(float& a0, float& a1, uint32_t v0, uint32_t v1, float s) {
    unsigned long long acc, v, sc;
    asm("mov.b64 %0, {%1, %2};" : "=l"(acc) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(v0), "r"(v1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(s));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(v), "l"(sc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Output element types of the fused epilogues: the cast-on-store modes of the reference's fix pipe (float32 ->
// bf16 / half / float32: include/tensor_api/impl/tensor_api/arch/cube/utils/l0c2out_utils.h:122-132).
// OUT_MX_E4M3 is the fused quantising output: E4M3 codes plus one E8M0 scale byte per 32 consecutive columns of a row,
// the operand format of the next MX GEMM (the reference plans this as its epilogue extension:
// docs/API/epilogue/block/block_epilogue.md:133; fix-pipe FP8 quant modes l0c2out_utils.h:75-76).
// OUT_FP8_128 is its counterpart in the FP8 kernel: E4M3 codes plus one float32 scale (amax / 448) per 128 columns.
enum OutType : int { OUT_BF16 = 0, OUT_F16 = 1, OUT_F32 = 2, OUT_MX_E4M3 = 3, OUT_FP8_128 = 4 };

// Four floats -> four E4M3 bytes (x in the low byte), round-to-nearest-even, saturating.
__device__ __forceinline__ uint32_t cvt_e4m3x4_sat(float x, float y, float z, float w) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(z, w), __NV_SATFINITE, __NV_E4M3);
    return (lo & 0xFFFFu) | (hi << 16);
}

}  // namespace blaze
