// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention
// kernels use: mbarrier with bounded waits, plain TMA tile loads (each CTA loads
// its own tiles), tcgen05 tensor-memory allocation, MMA issue, commit, and
// tensor-memory loads/stores, plus the shared-memory / instruction descriptor
// encoders for bf16 operands in 128-byte-swizzled tiles.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace dscuda {
namespace sm100 {

// ---------------------------------------------------------------------------
// Device status word.  A wait that runs out sets it; every kernel in the same
// translation unit checks it on entry and leaves at once when it is set, so a
// broken pipeline costs one time limit, not one per CTA.
// ---------------------------------------------------------------------------
enum DeviceStatus : int {
    STATUS_OK = 0,
    STATUS_WAIT_TIMEOUT = 1,
    STATUS_SMEM_MISALIGNED = 2,    // a kernel that cannot realign found its dynamic shared memory off a 1024-byte boundary
    STATUS_BAD_INDEX = 3,          // a page number or position outside the cache was skipped
};

// Roughly 0.1 s at 2 GHz; far above any legitimate wait (microseconds).
constexpr long long WAIT_LIMIT_CYCLES = 200LL * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ uint32_t lane_id() {
    return threadIdx.x & 31U;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking probe of the same condition.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete.  Gives up when
// `limit_cycles` of clock64 time have passed or when another thread of the CTA
// has already given up (`abort_flag`, in shared memory); then it raises both
// flags and returns false, and the caller must leave its loop and go to the
// common teardown.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word,
                                                long long limit_cycles) {
    if (mbar_test_wait(bar, parity)) {
        return true;
    }
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((spin & 31U) == 0U) {
            if (*abort_flag != 0 || clock64() - start > limit_cycles) {
                *abort_flag = 1;
                atomicExch(status_word, STATUS_WAIT_TIMEOUT);
                return false;
            }
        }
    }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word) {
    return mbar_wait_limit(bar, parity, abort_flag, status_word, WAIT_LIMIT_CYCLES);
}

// Register re-distribution between warpgroups (all four warps of a warpgroup
// must execute the same one).
template <int REGISTERS>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

template <int REGISTERS>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

// ---------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA: 2-D tile load global -> shared, completion on an mbarrier.  Plain
// per-CTA form only.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tensor_map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(tensor_map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const void* tensor_map, uint32_t bar, int x, int y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_dst), "l"(tensor_map), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// 3-D form: coordinates {x (element), y (row), z (chunk)}.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const void* tensor_map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_dst), "l"(tensor_map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// TMA tile store shared -> global (rows / columns outside the tensor are clipped), tracked by bulk groups.
__device__ __forceinline__ void tma_store_2d(const void* tensor_map, uint32_t smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tensor_map), "r"(smem_src), "r"(x), "r"(y) : "memory");
}

// A cache policy for data that is written or read once: first in line for eviction from L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void tma_store_2d_hint(const void* tensor_map, uint32_t smem_src, int x, int y, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(tensor_map), "r"(smem_src), "r"(x),
                 "r"(y), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Returns once the stores committed so far have read their shared-memory source.
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Returns once the stores committed so far are complete (written).
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---------------------------------------------------------------------------
// Tensor memory
// ---------------------------------------------------------------------------
// One full warp allocates `columns` (power of two, 32..512); the base address
// is written to shared memory at `smem_result`.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns) : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 bit, N consecutive columns per thread: thread i of warp w reads
// lane 32*(w%4)+i.  `taddr` holds lane<<16 | column.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 MMA issue
// ---------------------------------------------------------------------------
// Warp-uniform issue: the whole warp runs the issue loop (waits, address arithmetic, loop
// control) and the lane picked by elect_one() executes the tcgen05 instruction.  Measured on
// B200: an issue loop inside `if (lane == 0)` delivers a 128x128x16 MMA every 86 cycles with the
// other warps idle and every 120-245 cycles while they compute; the same loop run by the whole
// warp with a predicated MMA delivers one every 64-86 cycles (64 is the tensor core's rate).
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t leader;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(leader));
    return leader;
}

// D[tmem] (+)= A[smem] * B[smem], executed by the lane with `leader` != 0.
__device__ __forceinline__ void mma_ss_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                             uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A is K-major: lane = row, two bf16 per column.
__device__ __forceinline__ void mma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                             uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

// Makes `bar` complete one arrival once every MMA the elected lane has issued so far has
// finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit_elect(uint32_t bar, uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(bar), "r"(leader)
        : "memory");
}

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D.
//   bits 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format,
//   15 A major (0 = K), 16 B major (0 = K, 1 = MN), 17-22 N>>3, 24-28 M>>4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1U << 4) | (1U << 7) | (1U << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.
//   bits 0-13 address>>4, 16-29 leading byte offset>>4, 32-45 stride byte
//   offset>>4, 46-47 version (1 on sm_100), 61-63 layout (2 = 128B swizzle).
//
// K-major operand (rows of 64 bf16 = 128 B, 8-row groups of 1024 B): the
// leading offset is unused (1), the stride offset is the distance between
// 8-row groups.  Stepping 16 elements along K inside the 128-byte row adds
// 32 bytes to the start address.
//
// MN-major operand (each K index is a 128-byte row of 64 consecutive MN
// elements, 8 K indices per 1024-byte group): the leading offset is the
// distance between 64-element MN blocks, the stride offset the distance
// between 8-K groups.  Stepping 16 along K adds 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFU) >> 4) |
           (static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFU) << 16) |
           (static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFU) << 32) |
           (1ULL << 46) | (2ULL << 61);
}

// The same without a swizzle, for an MN-major operand stored as core matrices of 8 K indices x 16 bytes
// (8 consecutive MN elements), 128 contiguous bytes each: the leading offset is the distance between core
// matrices along K, the stride offset the distance between core matrices along MN.
__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFU) >> 4) |
           (static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFU) << 16) |
           (static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFU) << 32) |
           (1ULL << 46);
}

__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr) {
    return make_smem_desc(smem_addr, 16, 1024);
}

// Split form of the descriptor for issue loops: the high word is a compile-time
// constant per operand kind, the low word is (address >> 4) | leading offset and
// advances by (bytes >> 4) with a plain 32-bit add.
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t stride_bytes) {
    return ((stride_bytes >> 4) & 0x3FFFU) | (1U << 14) | (2U << 29);
}

__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr, uint32_t leading_bytes) {
    return ((smem_addr & 0x3FFFFU) >> 4) | (((leading_bytes >> 4) & 0x3FFFU) << 16);
}

// Elected-lane forms of the split-descriptor MMAs (see elect_one()).
__device__ __forceinline__ void mma_ss_split_elect(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                   uint32_t idesc, uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void mma_ts_split_elect(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                   uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

// Packed fp32 pairs (sm_100): two FMAs / adds per instruction.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra;
    asm("{\n\t"
        ".reg .b64 x, y, z;\n\t"
        "mov.b64 x, {%1, %2};\n\t"
        "mov.b64 y, {%3, %4};\n\t"
        "mov.b64 z, {%5, %6};\n\t"
        "fma.rn.f32x2 %0, x, y, z;\n\t"
        "}\n"
        : "=l"(ra)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    float2 result;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(result.x), "=f"(result.y) : "l"(ra));
    return result;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra;
    asm("{\n\t"
        ".reg .b64 x, y;\n\t"
        "mov.b64 x, {%1, %2};\n\t"
        "mov.b64 y, {%3, %4};\n\t"
        "add.rn.f32x2 %0, x, y;\n\t"
        "}\n"
        : "=l"(ra)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    float2 result;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(result.x), "=f"(result.y) : "l"(ra));
    return result;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float result;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(result) : "f"(a), "f"(b), "f"(c));
    return result;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace sm100
}  // namespace dscuda
