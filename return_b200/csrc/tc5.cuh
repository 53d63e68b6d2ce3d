// Blackwell (sm_100a) fifth-generation tensor-core primitives as thin inline-PTX wrappers:
// tensor memory (TMEM) allocation, tcgen05.mma issued by one thread with operands described by
// shared-memory descriptors, tcgen05.commit onto an mbarrier, tcgen05.ld of accumulators, and the
// mbarrier / proxy fences that order them.  Every wait is bounded: a wait that gives up sets an
// error flag and lets the kernel run to its end (it frees its TMEM and returns), so a fault in a
// descriptor shows as a wrong result and a status word, never as a hung GPU.
#pragma once

#include "common.cuh"

namespace tc5 {

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity; gives up after ~a second's worth of polls.
// Returns false (and the caller raises the kernel's error flag) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned spin = 0; spin < (1u << 24); ++spin) {
        unsigned done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// generic-proxy writes to shared memory (st.shared, cp.async) become visible to the async proxy
// (tcgen05.mma operand reads, TMA) after this fence
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------- tensor memory
// One warp allocates `cols` columns (a power of two, 32..512); the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(unsigned slot_smem, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------- operands
// A tile in shared memory for a K-major operand (rows x 64 bf16, i.e. 128 bytes a row) in the
// 128-byte-swizzled canonical layout: groups of 8 rows are 1024 bytes apart, a row is 128 bytes, and
// the 16-byte chunk c of row r sits at chunk (c ^ (r & 7)).  The tile base is 1024-byte aligned.
__device__ __forceinline__ unsigned sw128_offset(int row, int chunk) {
    return (unsigned)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// Shared-memory matrix descriptor of such a tile, starting `k_byte_offset` bytes into a row (the
// k16 step inside the 64-wide slab): start address, stride between 8-row groups (1024 B),
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned tile_smem_addr, unsigned k_byte_offset) {
    unsigned long long d = 0;
    d |= (unsigned long long)(((tile_smem_addr + k_byte_offset) & 0x3FFFFu) >> 4);        // [0,14) start address
    d |= (unsigned long long)(0u) << 16;                                                   // [16,30) leading byte offset: unused here
    d |= (unsigned long long)(1024u >> 4) << 32;                                           // [32,46) stride byte offset
    d |= 1ull << 46;                                                                       // [46,48) version
    d |= 2ull << 61;                                                                       // [61,64) SWIZZLE_128B
    return d;
}

// The same tile read as an MN-major operand (the 128-byte rows run along M or N, successive rows
// along K): `lead` bytes between blocks of 64 elements along M/N, `stride` bytes between groups of
// 8 rows along K.
__device__ __forceinline__ unsigned long long smem_desc_sw128_mn(unsigned start_smem_addr, unsigned lead, unsigned stride) {
    unsigned long long d = 0;
    d |= (unsigned long long)((start_smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lead >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((stride >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> f32, tile M x N.  A is K-major; B is K-major,
// or MN-major (its rows run along N) with b_mn_major.
__device__ __forceinline__ unsigned instr_desc_bf16(int M, int N, bool b_mn_major = false) {
    unsigned d = 0;
    d |= 1u << 4;                       // accumulator format: f32
    d |= 1u << 7;                       // A format: bf16
    d |= 1u << 10;                      // B format: bf16
    d |= (b_mn_major ? 1u : 0u) << 16;  // B major: 0 K, 1 MN
    d |= (unsigned)(N >> 3) << 17;      // N / 8
    d |= (unsigned)(M >> 4) << 24;      // M / 16
    return d;
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void mma_ss(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((unsigned)accumulate) : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace tc5
