// Device-side building blocks shared by the decode and prefill kernels:
// bf16 rounding helpers, warp reductions, bounded mbarrier waits, 1-D bulk
// async copies (TMA, non-multicast) and programmatic-dependent-launch control.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megaqwen_b200.h"

namespace mq {

constexpr int H = MQ_HIDDEN;
constexpr int I = MQ_INTERMEDIATE;
constexpr int NQ = MQ_NUM_Q_HEADS;
constexpr int NKV = MQ_NUM_KV_HEADS;
constexpr int D = MQ_HEAD_DIM;
constexpr int QSZ = MQ_Q_SIZE;
constexpr int KVSZ = MQ_KV_SIZE;
constexpr int QKV = QSZ + 2 * KVSZ;
constexpr float RMS_EPS = 1e-6f;

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------- rounding
// Every value that the HuggingFace bf16 model materialises as a tensor is
// rounded to bf16 here too; these helpers make the rounding points explicit.
__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
// silu evaluated in fp32 as x / (1 + exp(-x)), rounded to bf16 by the caller.
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ unsigned int warp_sum_u32(unsigned int v) { return __reduce_add_sync(0xffffffffu, v); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---------------------------------------------------------------- loads
// Activations are rewritten by every kernel of the chain while kernels overlap
// under programmatic dependent launch, so they are always read through L2
// (ld.global.cg), never through a possibly stale L1 line.
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ld_cg_u2(const void* p) { return __ldcg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) { return __ldcg(reinterpret_cast<const uint32_t*>(p)); }
__device__ __forceinline__ int ld_cg_i32(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_cg_f32(const float* p) { return __ldcg(p); }

// ---------------------------------------------------------------- PDL
// griddepcontrol.wait: block until every grid this one depends on has
// completed and its memory is visible.  launch_dependents: allow the next
// kernel of the stream to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The whole CTA waits for the preceding grid, but only warp 0 executes the wait; the other
// warps sleep on the block barrier.  Warps parked in griddepcontrol.wait compete for issue
// slots with the co-resident CTA of the running kernel (three waiting CTAs of eight warps
// each made its dependent mma loop three times slower).
__device__ __forceinline__ void pdl_wait_cta() {
    if (threadIdx.x < 32) pdl_wait();
    __syncthreads();
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- mbarrier + bulk copy
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
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

// Bounded wait (about 0.2 s of SM clock).  On expiry the sticky status bit is
// set and the caller carries on with whatever the buffer holds: the kernel
// finishes, the host sees the bit at its next status check, and the GPU stays
// usable.  Once the bit is set every later wait gives up after a few dozen
// polls, so a broken chain drains quickly instead of paying one timeout per
// wait.  Returns false if the wait was abandoned.
constexpr long long WAIT_LIMIT_CYCLES = 400000000LL;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    // The sticky word lives in global memory (an L2 round trip): it is looked at every 64 polls, not
    // before the first one, where it would sit in front of every wait that is not
    // already satisfied (a producer waiting for a free stage, the first tiles of a pipeline).
    const long long t0 = clock64();
    int polls = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++polls & 63) == 0) {
            if (status && (__ldcg(status) & MQ_STATUS_WAIT_TIMEOUT)) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                if (status) atomicOr(status, MQ_STATUS_WAIT_TIMEOUT);
                return false;
            }
        }
    }
    return true;
}

// 1-D bulk async copy global -> this CTA's shared memory, completing `bytes`
// on `bar`.  Both addresses 16-byte aligned, bytes a multiple of 16.  No
// cluster multicast.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------- dot products
// A warp multiplies one 1024-wide slice of a bf16 weight row held in shared
// memory with a slice of the activation vector held in registers.  Lane l owns
// columns j*256 + l*8 + e (j < 4, e < 8): each lane reads 16 contiguous bytes,
// a warp 512 contiguous bytes, so the loads are bank-conflict free.
__device__ __forceinline__ void load_x_slice(float (&x)[32], const bf16* src, int lane) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint4 u = ld_cg_u4(src + j * 256 + lane * 8);
        x[j * 8 + 0] = bf_lo(u.x); x[j * 8 + 1] = bf_hi(u.x);
        x[j * 8 + 2] = bf_lo(u.y); x[j * 8 + 3] = bf_hi(u.y);
        x[j * 8 + 4] = bf_lo(u.z); x[j * 8 + 5] = bf_hi(u.z);
        x[j * 8 + 6] = bf_lo(u.w); x[j * 8 + 7] = bf_hi(u.w);
    }
}

// Asks the L2 to fetch bytes (a multiple of 16) that a later kernel will copy to shared memory.
__device__ __forceinline__ void l2_prefetch(const void* g, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(g), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------- tensor-core GEMV
// The per-layer decode kernels multiply a handful of weight rows (in shared memory) with
// one activation vector.  Done with fp32 FMAs this takes about a thousand straight-line
// instructions per warp, and a kernel that runs its code exactly once is bound by
// instruction fetch; mma.sync m16n8k16 does sixteen rows x sixteen columns per
// instruction in a short loop.  The vector is replicated over the eight B columns, so
// every column of the accumulator holds the same sixteen dot products.
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
// ---- FP8 (e4m3) KV cache: the attention kernels multiply f16 tiles (every e4m3 value is exact
// in f16) with the same fragment layouts as the bf16 tiles.
__device__ __forceinline__ void mma16816_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool F16>
__device__ __forceinline__ void mma16816_sel(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (F16) mma16816_f16(c, a, b0, b1);
    else mma16816(c, a, b0, b1);
}
// four e4m3 bytes (little endian) -> four f16 (lo = elements 0, 1; hi = elements 2, 3)
__device__ __forceinline__ void fp8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
    asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; cvt.rn.f16x2.e4m3x2 %0, l; cvt.rn.f16x2.e4m3x2 %1, h; }" : "=r"(lo), "=r"(hi) : "r"(w));
}
// sixteen e4m3 bytes -> sixteen f16 (two 16-byte words)
__device__ __forceinline__ void fp8x16_to_f16x16(const uint4& w, uint4& a, uint4& b) {
    fp8x4_to_f16x4(w.x, a.x, a.y);
    fp8x4_to_f16x4(w.y, a.z, a.w);
    fp8x4_to_f16x4(w.z, b.x, b.y);
    fp8x4_to_f16x4(w.w, b.z, b.w);
}
// round-to-nearest-even, saturating at +-448 (the conversion of __nv_fp8_e4m3(float)); hi -> upper byte
__device__ __forceinline__ uint32_t f32x2_to_fp8x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}
__device__ __forceinline__ uint32_t f32x4_to_fp8x4(float a, float b, float c, float d) {
    return f32x2_to_fp8x2(a, b) | (f32x2_to_fp8x2(c, d) << 16);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// the scale a quantised cache is read with: amax / 448, or 1 for an all-zero span
// (reference: kv_fp8_max_abs_scale, csrc/megakernel/split_decode_gemm.cu:74-78)
__host__ __device__ __forceinline__ float kv_fp8_scale_of(float amax) { return amax < 1.0e-8f ? 1.0f : amax / 448.0f; }
// a stored scale below 1e-8 reads as 1 (split_decode_gemm.cu:445-446)
__device__ __forceinline__ float kv_fp8_scale_guard(float s) { return s < 1.0e-8f ? 1.0f : s; }

// 16-byte asynchronous copies global -> shared (any shared address: padded rows)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}

// Rows live in shared memory with a stride of K + 8 elements (16 bytes of padding), which
// spreads the eight 16-byte rows of an ldmatrix over all banks.  Lane l addresses row
// (l & 15) of a tile at column offset 8 * (l >> 4).  rowaddr[t] is that lane's byte address
// for tile t at column 0; the warp accumulates k-steps [ks0, ks1) of 16 columns each.
// Lanes 0, 4, .., 28 end with row l/4 in c[t][0] and row l/4 + 8 in c[t][2].
template <int NT>
__device__ __forceinline__ void mma_gemv(const uint32_t (&rowaddr)[NT], uint32_t xs_addr, int ks0, int ks1, int lane, float (&c)[NT][4]) {
    const uint32_t xb = xs_addr + (uint32_t)(lane & 3) * 4u;
#pragma unroll 2
    for (int ks = ks0; ks < ks1; ++ks) {
        const uint32_t b0 = lds32(xb + (uint32_t)ks * 32u), b1 = lds32(xb + (uint32_t)ks * 32u + 16u);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            uint32_t a[4];
            ldsm4(a, rowaddr[t] + (uint32_t)ks * 32u);
            mma16816(c[t], a, b0, b1);
        }
    }
}

__device__ __forceinline__ float dot_slice(const bf16* wrow_smem, const float (&x)[32], int lane) {
    const uint4* w4 = reinterpret_cast<const uint4*>(wrow_smem);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint4 u = w4[j * 32 + lane];
        a0 = fmaf(bf_lo(u.x), x[j * 8 + 0], a0); a1 = fmaf(bf_hi(u.x), x[j * 8 + 1], a1);
        a0 = fmaf(bf_lo(u.y), x[j * 8 + 2], a0); a1 = fmaf(bf_hi(u.y), x[j * 8 + 3], a1);
        a0 = fmaf(bf_lo(u.z), x[j * 8 + 4], a0); a1 = fmaf(bf_hi(u.z), x[j * 8 + 5], a1);
        a0 = fmaf(bf_lo(u.w), x[j * 8 + 6], a0); a1 = fmaf(bf_hi(u.w), x[j * 8 + 7], a1);
    }
    return a0 + a1;
}

// RMSNorm of a 1024-wide bf16 vector held as a register slice per lane (every
// warp holds the whole vector): x <- bf16(w * bf16(x * rsqrt(mean(x^2) + eps))).
__device__ __forceinline__ void rmsnorm_slice(float (&x)[32], const bf16* w, int lane) {
    uint4 wu[4];   // requested before the row sum, used after it
#pragma unroll
    for (int j = 0; j < 4; ++j) wu[j] = *reinterpret_cast<const uint4*>(w + j * 256 + lane * 8);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 u = wu[j];
        const float wv[8] = {bf_lo(u.x), bf_hi(u.x), bf_lo(u.y), bf_hi(u.y), bf_lo(u.z), bf_hi(u.z), bf_lo(u.w), bf_hi(u.w)};
#pragma unroll
        for (int e = 0; e < 8; ++e) x[j * 8 + e] = rbf(wv[e] * rbf(x[j * 8 + e] * r));
    }
}

}  // namespace mq
