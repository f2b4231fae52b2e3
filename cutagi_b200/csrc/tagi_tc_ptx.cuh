// Thin inline-PTX layer for the sm_100a tensor-core path: mbarriers, TMA tile loads,
// tensor-memory allocation, tcgen05 MMA / commit / load, and the descriptor encodings.
// Every wait is bounded: after the limit it raises the CTA's abort flag and records a
// status code, so a protocol error ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace tagi {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
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

// Non-blocking test: for the single producer / issuer threads, whose wake-up latency paces the pipeline
// (try_wait may park the thread for a while before it looks again).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Status codes written to the device status word when a wait runs out.
enum { ST_OK = 0, ST_TIMEOUT_EMPTY = 1, ST_TIMEOUT_RAW = 2, ST_TIMEOUT_CONV = 3, ST_TIMEOUT_ACC = 4 };

// Wait for a phase with a cycle limit (about one second at 2 GHz). Returns false when the CTA is
// aborting, either because this wait ran out or because another thread's did.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        // the abort flag lives in shared memory: look at it rarely so that polling does not eat LSU bandwidth
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 2000000000LL) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// Same bounded wait, spinning on test_wait (lowest wake-up latency; use from single threads only).
__device__ __forceinline__ bool mbar_spin(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((spin & 1023u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 2000000000LL) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// ----------------------------------------------------------------------------- cp.async (4-byte gathers)
// Copies 4 bytes global -> shared asynchronously; `valid` false writes zero and reads nothing.
__device__ __forceinline__ void cp_async_f32(uint32_t smem_dst, const float *src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(src), "r"(valid ? 4 : 0) : "memory");
}
// The barrier receives one arrival (already counted in its init count) when all cp.async of this thread so far are done
__device__ __forceinline__ void cp_async_arrive(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ----------------------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ----------------------------------------------------------------------------- TMA
// 2-D tiled load; x is the coordinate along the contiguous dimension (x * 4 bytes must be a multiple of 16).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// 4-D tiled load (x innermost); same alignment rule for x. Coordinates outside the tensor read the fill value (zero).
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const void *tmap, int x, int y, int z, int w, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(smem_dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ----------------------------------------------------------------------------- tensor memory
// Executed by one whole warp. ncols is a power of two >= 32. The base address lands in *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
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
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 8 consecutive 32-bit columns written from registers: thread i of the warp writes row (lane base + i).
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const float (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                 "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
                 "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (64 bit): start address, leading / stride byte offsets (all >> 4),
// version 1 (bits 46-47), swizzle mode in bits 61-63.
enum { SWZ_NONE = 0, SWZ_128B_BASE32B = 1, SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6 };
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)swizzle << 61;
    return d;
}

// Instruction descriptor for kind::tf32, FP32 accumulation: c_format F32 (bits 4-5 = 1), a/b format TF32
// (bits 7-9 / 10-12 = 2), a_major bit 15, b_major bit 16 (1 = MN-major), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A is M x 8 in tensor memory (lane = row, one tf32 per 32-bit column).
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on an mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ----------------------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster drive one tensor-core instruction of 256 rows: each holds 128 rows of A / D in its own tensor
// memory and half of B's rows in its own shared memory. One thread of the even CTA issues; completion is signalled to
// barriers in both CTAs.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster (release at cluster scope)
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t *bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(smem_u32(bar)), "r"(cta)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.relaxed.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait with cluster-scope acquire (the arrivals come from both CTAs of the pair)
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status,
                                                  int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 2000000000LL) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem, both CTAs] (+)= A[tmem, both CTAs] * B[smem halves of both CTAs]; M = 256
__device__ __forceinline__ void mma_tf32_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// completion of every MMA issued so far -> arrive on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}

// ----------------------------------------------------------------------------- batched MMA issue
// The thread that issues the MMAs is the pacemaker of the whole CTA: measured on the B200, building every
// descriptor in C++ and issuing the MMAs one asm statement at a time cost ~90 cycles per MMA of issue time against
// 56 cycles of tensor-core time. The groups below issue all MMAs of one 8-wide k step in a single asm block: the
// high descriptor word is constant, the low word is a base plus a literal tile offset, the predicates are set once.
//   at   : tensor-memory address of A tile 0 for this k step (tile i is 16 columns further)
//   rbl  : low descriptor word of raw B tile 0 for this k step, dsl: of derived B tile 0; tile i is BS units of 16 bytes on
//   hi   : high descriptor word (stride offset, version, swizzle)
//   f1/f2: 0 -> the first MMA into D1 / D2 overwrites (start of an accumulation chunk), else accumulates
#define TAGI_STR_(x) #x
#define TAGI_STR(x) TAGI_STR_(x)
#define TAGI_MMA_HEAD                                             \
    "{\n\t.reg .pred p1, p2, pt;\n\t.reg .b32 ta, tb;\n\t.reg .b64 db;\n\t" \
    "setp.ne.b32 p1, %7, 0;\n\tsetp.ne.b32 p2, %8, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
// one MMA: D operand index, A tile, B base operand index (3 = raw, 4 = derived), B tile, predicate
#define TAGI_MMA(CG, D, AT, BB, BT, BS, P)                                          \
    "add.u32 ta, %2, " TAGI_STR(AT) " * 16;\n\t"                                    \
    "add.u32 tb, %" #BB ", " TAGI_STR(BT) " * " TAGI_STR(BS) ";\n\t"                \
    "mov.b64 db, {tb, %5};\n\t"                                                     \
    "tcgen05.mma.cta_group::" #CG ".kind::tf32 [%" #D "], [ta], db, %6, " #P ";\n\t"
#define TAGI_MMA_OPERANDS \
    ::"r"(d1), "r"(d2), "r"(at), "r"(rbl), "r"(dsl), "r"(hi), "r"(idesc), "r"(f1), "r"(f2) : "memory"

// Measured on the B200: one thread issues at most one tcgen05.mma per ~50-56 cycles whatever the MMA's size, and two
// warps issue concurrently at twice that rate. A 128 x 112 x 8 MMA takes 56 tensor-core cycles, so a single issuing
// thread has no slack for anything else; the MMAs are therefore split by accumulator between two issuing warps
// (chain 1 = everything that accumulates into D1, chain 2 = D2), which also means no accumulator is shared between
// issuers and no ordering between them is needed.
// forward: A tiles 0 mu_a, 1 var_a, 2 mu_a lo, 3 var_a lo, 4 S, 5 S lo ; raw B 0 mu_w, 1 var_w ; derived B 0 mu_w lo,
// 1 var_w lo, 2 Q, 3 Q lo.  D1 = mu_a.mu_w ; D2 = S.var_w + var_a.Q, each as hi*hi + hi*lo + lo*hi
#define TAGI_MMA_D1(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMA(CG, 0, 0, 3, 0, BS, p1) TAGI_MMA(CG, 0, 0, 4, 0, BS, pt) TAGI_MMA(CG, 0, 2, 3, 0, BS, pt) "}"
#define TAGI_MMA_FWD_D2(CG, BS)                                                                                   \
    TAGI_MMA_HEAD TAGI_MMA(CG, 1, 4, 3, 1, BS, p2) TAGI_MMA(CG, 1, 1, 4, 2, BS, pt) TAGI_MMA(CG, 1, 4, 4, 1, BS, pt) \
        TAGI_MMA(CG, 1, 5, 3, 1, BS, pt) TAGI_MMA(CG, 1, 1, 4, 3, BS, pt) TAGI_MMA(CG, 1, 3, 4, 2, BS, pt) "}"
// backward: A tiles 0 a0, 1 a1, 2 a0 lo, 3 a1 lo ; raw B 0 w ; derived B 0 w lo, 1 Q = w^2, 2 Q lo.  D1 = a0.w (same
// three MMAs as the forward D1) ; D2 = a1.Q
#define TAGI_MMA_BWD_D2(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMA(CG, 1, 1, 4, 1, BS, p2) TAGI_MMA(CG, 1, 1, 4, 2, BS, pt) TAGI_MMA(CG, 1, 3, 4, 1, BS, pt) "}"

// Conv2d parameter pass with the roles swapped (tagi_conv_patch.cu): A tiles 0 x, 1 q = x^2, 2 x lo, 3 q lo ; raw B 0 dmu,
// 1 dvar ; derived B 0 dmu lo, 1 dvar lo.  D1 = x.dmu (the three MMAs of TAGI_MMA_D1) ; D2 = q.dvar
#define TAGI_MMA_CPARAM_D2(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMA(CG, 1, 1, 3, 1, BS, p2) TAGI_MMA(CG, 1, 1, 4, 1, BS, pt) TAGI_MMA(CG, 1, 3, 3, 1, BS, pt) "}"

// The same chains with 32-wide k slabs: A tiles 32 tensor-memory columns apart, B tiles BS units of 16 bytes apart
#define TAGI_MMAW(CG, D, AT, BB, BT, BS, P)                                         \
    "add.u32 ta, %2, " TAGI_STR(AT) " * 32;\n\t"                                    \
    "add.u32 tb, %" #BB ", " TAGI_STR(BT) " * " TAGI_STR(BS) ";\n\t"                \
    "mov.b64 db, {tb, %5};\n\t"                                                     \
    "tcgen05.mma.cta_group::" #CG ".kind::tf32 [%" #D "], [ta], db, %6, " #P ";\n\t"
#define TAGI_MMAW_D1(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMAW(CG, 0, 0, 3, 0, BS, p1) TAGI_MMAW(CG, 0, 0, 4, 0, BS, pt) TAGI_MMAW(CG, 0, 2, 3, 0, BS, pt) "}"
#define TAGI_MMAW_CPARAM_D2(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMAW(CG, 1, 1, 3, 1, BS, p2) TAGI_MMAW(CG, 1, 1, 4, 1, BS, pt) TAGI_MMAW(CG, 1, 3, 3, 1, BS, pt) "}"
#define TAGI_MMAW_FWD_D2(CG, BS)                                                                                      \
    TAGI_MMA_HEAD TAGI_MMAW(CG, 1, 4, 3, 1, BS, p2) TAGI_MMAW(CG, 1, 1, 4, 2, BS, pt) TAGI_MMAW(CG, 1, 4, 4, 1, BS, pt) \
        TAGI_MMAW(CG, 1, 5, 3, 1, BS, pt) TAGI_MMAW(CG, 1, 1, 4, 3, BS, pt) TAGI_MMAW(CG, 1, 3, 4, 2, BS, pt) "}"
#define TAGI_MMAW_BWD_D2(CG, BS) \
    TAGI_MMA_HEAD TAGI_MMAW(CG, 1, 1, 4, 1, BS, p2) TAGI_MMAW(CG, 1, 1, 4, 2, BS, pt) TAGI_MMAW(CG, 1, 3, 4, 1, BS, pt) "}"

// CHAIN 1 or 2; BS = 512: B tiles of 8 KiB (one CTA); BS = 256: B half tiles of 4 KiB (CTA pairs, cta_group::2)
template <bool FWD, int CHAIN>
__device__ __forceinline__ void mma_kstep_ts(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl, uint32_t hi,
                                             uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (CHAIN == 1) asm volatile(TAGI_MMA_D1(1, 512) TAGI_MMA_OPERANDS);
    else if (FWD) asm volatile(TAGI_MMA_FWD_D2(1, 512) TAGI_MMA_OPERANDS);
    else asm volatile(TAGI_MMA_BWD_D2(1, 512) TAGI_MMA_OPERANDS);
}
template <bool FWD, int CHAIN>
__device__ __forceinline__ void mma_kstep_pair(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl,
                                               uint32_t hi, uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (CHAIN == 1) asm volatile(TAGI_MMA_D1(2, 256) TAGI_MMA_OPERANDS);
    else if (FWD) asm volatile(TAGI_MMA_FWD_D2(2, 256) TAGI_MMA_OPERANDS);
    else asm volatile(TAGI_MMA_BWD_D2(2, 256) TAGI_MMA_OPERANDS);
}
template <int CHAIN>
__device__ __forceinline__ void mma_kstep_cparam_pair(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl,
                                                      uint32_t hi, uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (CHAIN == 1) asm volatile(TAGI_MMA_D1(2, 256) TAGI_MMA_OPERANDS);
    else asm volatile(TAGI_MMA_CPARAM_D2(2, 256) TAGI_MMA_OPERANDS);
}
// The same k steps issued by one CTA for itself (cta_group::1, 128 rows), B tiles 4 KiB apart as in the pair kernels
template <int CHAIN>
__device__ __forceinline__ void mma_kstep_cparam_solo(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl,
                                                      uint32_t hi, uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (CHAIN == 1) asm volatile(TAGI_MMA_D1(1, 256) TAGI_MMA_OPERANDS);
    else asm volatile(TAGI_MMA_CPARAM_D2(1, 256) TAGI_MMA_OPERANDS);
}
template <bool FWD, int CHAIN>
__device__ __forceinline__ void mma_kstep_solo(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl,
                                               uint32_t hi, uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (CHAIN == 1) asm volatile(TAGI_MMA_D1(1, 256) TAGI_MMA_OPERANDS);
    else if (FWD) asm volatile(TAGI_MMA_FWD_D2(1, 256) TAGI_MMA_OPERANDS);
    else asm volatile(TAGI_MMA_BWD_D2(1, 256) TAGI_MMA_OPERANDS);
}
// 32-wide k slabs: one 8-wide k step; PAIR selects cta_group::2; B tiles 8 KiB apart
template <bool PAIR, int CHAIN>
__device__ __forceinline__ void mma_kstep_cparam_w(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl,
                                                   uint32_t hi, uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (PAIR) {
        if (CHAIN == 1) asm volatile(TAGI_MMAW_D1(2, 512) TAGI_MMA_OPERANDS);
        else asm volatile(TAGI_MMAW_CPARAM_D2(2, 512) TAGI_MMA_OPERANDS);
    } else {
        if (CHAIN == 1) asm volatile(TAGI_MMAW_D1(1, 512) TAGI_MMA_OPERANDS);
        else asm volatile(TAGI_MMAW_CPARAM_D2(1, 512) TAGI_MMA_OPERANDS);
    }
}
template <bool PAIR, bool FWD, int CHAIN>
__device__ __forceinline__ void mma_kstep_w(uint32_t d1, uint32_t d2, uint32_t at, uint32_t rbl, uint32_t dsl, uint32_t hi,
                                            uint32_t idesc, uint32_t f1, uint32_t f2) {
    if (PAIR) {
        if (CHAIN == 1) asm volatile(TAGI_MMAW_D1(2, 512) TAGI_MMA_OPERANDS);
        else if (FWD) asm volatile(TAGI_MMAW_FWD_D2(2, 512) TAGI_MMA_OPERANDS);
        else asm volatile(TAGI_MMAW_BWD_D2(2, 512) TAGI_MMA_OPERANDS);
    } else {
        if (CHAIN == 1) asm volatile(TAGI_MMAW_D1(1, 512) TAGI_MMA_OPERANDS);
        else if (FWD) asm volatile(TAGI_MMAW_FWD_D2(1, 512) TAGI_MMA_OPERANDS);
        else asm volatile(TAGI_MMAW_BWD_D2(1, 512) TAGI_MMA_OPERANDS);
    }
}
// low / high 32-bit words of a shared-memory matrix descriptor (see make_smem_desc)
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr >> 4) & 0x3fffu) | ((lbo_bytes >> 4) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes, uint32_t swizzle) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (swizzle << 29);
}

}  // namespace ptx
}  // namespace tagi
