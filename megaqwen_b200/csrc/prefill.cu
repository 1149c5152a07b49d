// Prefill (full-sequence forward) for sm_100a.
//
// The reference runs prefill as 7 cuBLAS GEMMs per layer plus ~14 small kernels
// and a serial-per-warp O(S^2) attention (csrc/megakernel/fused_prefill_launch.inl:71-731,
// fused_prefill_kernels.inl:3-824).  Here the dense contractions run on the
// 5th-generation tensor cores directly: one kernel per GEMM that stages both
// operands with TMA (128-byte swizzle) into a multi-stage shared-memory ring,
// issues tcgen05.mma from a single elected thread into a TMEM accumulator and
// drains it with tcgen05.ld in four epilogue warps, with the residual add and
// the SwiGLU product fused into the epilogue.  Activations are bf16 between
// all ops (the rounding points of the HF bf16 model, as in the reference's
// launch_prefill_float).
//
// Every mbarrier wait is bounded (mq_device.cuh) and TMEM is always freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "mq_device.cuh"

namespace mq {

// ---------------------------------------------------------------- tcgen05 / TMA primitives
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the A operand in tensor memory (row i of A in lane i, two consecutive K elements per 32-bit column)
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on `bar` once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes
// (64 elements) under the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* tile) {
    uint64_t d = (uint64_t)((smem_u32(tile) >> 4) & 0x3fffu);
    d |= 1ull << 16;                 // leading byte offset (unused for swizzled K-major), 16 B units
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= 1ull << 46;                 // descriptor version (sm_100)
    d |= 2ull << 61;                 // SWIZZLE_128B
    return d;
}

// The same tile read as an MN-major operand: [rows = K index][64 elements of the M / N dimension], i.e. a
// row-major [k][n] matrix used as B without transposing it.  A 128-byte row holds 64 consecutive n of one k;
// eight k form a 1024-byte swizzle group (stride byte offset); the next 64 n start panel_bytes further on
// (leading byte offset).  A K = 16 step advances the start address by two groups.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(const void* tile, uint32_t panel_bytes) {
    uint64_t d = (uint64_t)((smem_u32(tile) >> 4) & 0x3fffu);
    d |= (uint64_t)((panel_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Bounded wait that does not look at the sticky status word: used while a CTA drains after one of its
// waits has expired (copies already issued must land, MMAs already issued must finish, before the CTA
// hands back its shared and tensor memory).  About 1 ms.
__device__ __forceinline__ bool mbar_wait_drain(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > 2000000LL) return false;
    return true;
}

// ---------------------------------------------------------------- GEMM  C[M,N] = A[M,K] * B[N,K]^T
constexpr int GM_BM = 128;
constexpr int GM_BK = 64;
constexpr int GM_THREADS = 192;    // skinny GEMM: warp 0 TMA, warp 1 MMA + TMEM owner, warps 2..5 epilogue
// Tile GEMM: eight epilogue warps.  Warps w and w + 4 read the same quarter of the TMEM lanes (a warp may
// only touch lanes 32 (w % 4) .. + 31) and split the accumulator columns; with four warps the SwiGLU
// epilogue of a 256 x 256 tile (65 536 silu + products on 128 threads) took as long as its main loop.
constexpr int GM_EPI_WARPS = 8;
constexpr int GM_TILE_THREADS = 64 + 32 * GM_EPI_WARPS;
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3, EPI_STORE_2CTA = 4 };   // PARTIAL: fp32 plane blockIdx.z of a K split
// EPI_STORE_2CTA: EPI_STORE with a three-stage ring (97 KB), so that two CTAs share an SM.  For a GEMM of many short
// CTAs that stream weights (the batched LM head: 1187 column tiles of a 64-row matrix), where a lone CTA's start-up and
// epilogue leave the SM's memory pipeline idle.

// Every kernel of the prefill and batched-decode chains is launched with programmatic
// stream serialisation and begins with griddepcontrol.wait + launch_dependents: the next
// kernel's CTAs are scheduled (parameters loaded, shared memory carved) while this one runs,
// which takes the launch latency of the ~230 (prefill) / ~310 (batched step) kernels of a
// pass off the critical path.  Without the launch attribute both instructions are no-ops.
template <typename... KArgs, typename... Args>
static void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // errors are sticky: callers read cudaGetLastError()
}

#ifndef MQ_GEMM_BUDGET_KB
#define MQ_GEMM_BUDGET_KB 200   // shared memory for the operand ring of one CTA
#define MQ_GEMM_MIN_CTAS 1
#endif
// MT = 128-row A tiles per CTA.  With MT = 2 a CTA computes a 256-row output tile with two
// accumulators that share every B tile: the 128 x 128 tiles are bound by the operand traffic
// from the L2 into the SMs, and a 256-row tile moves a third less of it per FLOP.
template <int BN, int EPI, int MT = 1>
struct GemmCfg {
    static constexpr int NB = (EPI == EPI_SWIGLU) ? 2 : 1;                       // B operands per stage
    static constexpr int A_BYTES = MT * GM_BM * GM_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + NB * BN * GM_BK * 2;
    static constexpr int STAGES = EPI == EPI_STORE_2CTA ? 3 : (MQ_GEMM_BUDGET_KB * 1024) / STAGE_BYTES > 6 ? 6 : (MQ_GEMM_BUDGET_KB * 1024) / STAGE_BYTES;
    static constexpr int ACC_COLS = MT * NB * BN;                                // accumulator columns in use
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;   // allocations are powers of two
    static_assert(ACC_COLS <= 512 && BN % 32 == 0, "tensor memory holds 512 columns; the epilogue reads 32 at a time");
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

// x / (1 + e^-x) with the hardware exponential and reciprocal (2 ulp of fp32; the result is rounded to bf16)
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int BN, int EPI, int MT>
__global__ void __launch_bounds__(GM_TILE_THREADS, MQ_GEMM_MIN_CTAS)
k_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
       const __grid_constant__ CUtensorMap tmB3, int tiles0, int tiles1,
       bf16* __restrict__ C, const bf16* R, int M, int N, int K, int ldc, unsigned int* status, int drop_kb, int early_b) {
    // drop_kb >= 0 (test hook): the producer never requests k-block drop_kb, so the MMA thread's wait for it
    // runs out; -1 in every production launch.  early_b: B is constant over the stream's lifetime (a weight),
    // so its first tiles may be requested before the preceding grid has finished.
    pdl_trigger();   // the next grid may be scheduled already; it waits for this one below, after its own set-up
    // EPI_STORE / EPI_RESID may concatenate up to three B matrices along N (q|k|v): column tile
    // blockIdx.x < tiles0 reads tmB, < tiles0 + tiles1 tmB2, else tmB3.  EPI_SWIGLU uses tmB (gate)
    // and tmB2 (up) for the same tile.
    using Cfg = GemmCfg<BN, EPI, MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + Cfg::STAGES;
    uint64_t* accum = empty + Cfg::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    // Set by the thread whose bounded wait expired (the sticky status bit is then set as well).  Everybody
    // stops issuing work; the epilogue stores nothing; the CTA drains what is in flight before it exits.
    volatile uint32_t* aborted = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.y * GM_BM * MT, n0 = blockIdx.x * BN;
    // EPI_PARTIAL: gridDim.z CTAs share an output tile, each takes a contiguous range of k-blocks
    const int kb_first = (int)(((long long)blockIdx.z * (K / GM_BK)) / gridDim.z);
    const int nk = (int)(((long long)(blockIdx.z + 1) * (K / GM_BK)) / gridDim.z) - kb_first;
    const int tile = blockIdx.x;
    const CUtensorMap* mapB = &tmB;
    int brow0 = n0;
    if (EPI != EPI_SWIGLU && tile >= tiles0) {
        mapB = tile < tiles0 + tiles1 ? &tmB2 : &tmB3;
        brow0 = (tile < tiles0 + tiles1 ? tile - tiles0 : tile - tiles0 - tiles1) * BN;
    }

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (tid == 64) *aborted = 0u;       // by a thread that is idle now (thread 0's set-up gates the first TMA request)
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    // Barriers and tensor memory are set up while the preceding grid may still be running.  Where the B operand is
    // a weight matrix that nothing on the stream writes, its tiles for the first ring of stages are requested now
    // and cross HBM while that grid finishes; the A tiles (its output) follow the wait, from which on its results
    // are complete and visible.
    const int npre = !early_b ? 0 : nk < Cfg::STAGES ? nk : Cfg::STAGES;
    if (tid == 0) {
        for (int kb = 0; kb < npre; ++kb) {
            if (kb == drop_kb) continue;
            uint8_t* st = smem + (size_t)kb * Cfg::STAGE_BYTES;
            mbar_expect_tx(&full[kb], (uint32_t)Cfg::STAGE_BYTES);
            tma_load_2d(st + Cfg::A_BYTES, mapB, (kb_first + kb) * GM_BK, brow0, &full[kb]);
            if (EPI == EPI_SWIGLU) tma_load_2d(st + Cfg::A_BYTES + BN * GM_BK * 2, &tmB2, (kb_first + kb) * GM_BK, n0, &full[kb]);
        }
    }
    pdl_wait();

    int issued = npre;                    // k-blocks the producer has requested, B tiles at least (thread 0 only)
    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < nk; ++kb) {
                const int s = kb % Cfg::STAGES;
                if (kb >= Cfg::STAGES && !mbar_wait(&empty[s], (uint32_t)((kb / Cfg::STAGES) - 1) & 1u, status)) { *aborted = 1u; break; }
                if (*aborted) break;
                issued = kb + 1;
                if (kb == drop_kb) continue;
                uint8_t* st = smem + (size_t)s * Cfg::STAGE_BYTES;
                if (kb >= npre) mbar_expect_tx(&full[s], (uint32_t)Cfg::STAGE_BYTES);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) tma_load_2d(st + mt * GM_BM * GM_BK * 2, &tmA, (kb_first + kb) * GM_BK, m0 + mt * GM_BM, &full[s]);
                if (kb >= npre) {
                    tma_load_2d(st + Cfg::A_BYTES, mapB, (kb_first + kb) * GM_BK, brow0, &full[s]);
                    if (EPI == EPI_SWIGLU) tma_load_2d(st + Cfg::A_BYTES + BN * GM_BK * 2, &tmB2, (kb_first + kb) * GM_BK, n0, &full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = bf16, both K-major, N >> 3, M >> 4.  EPI_SWIGLU: the gate
            // and the up tile sit back to back in the stage (2 BN rows of one K-major operand), so ONE
            // instruction of N = 2 BN fills both accumulators (columns [0, BN) gate, [BN, 2 BN) up).  A
            // 128 x 128 x 16 instruction reads 8 KB of shared memory for 64 cycles of math, which is the
            // SM's whole shared-memory bandwidth; at N = 256 it is 12 KB for 128 cycles.
            constexpr int UMMA_N = Cfg::NB * BN;
            static_assert(UMMA_N <= 256, "one instruction spans at most 256 columns");
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(UMMA_N >> 3) << 17) | ((uint32_t)(GM_BM >> 4) << 24);
            for (int kb = 0; kb < nk; ++kb) {
                const int s = kb % Cfg::STAGES;
                if (!mbar_wait(&full[s], (uint32_t)(kb / Cfg::STAGES) & 1u, status)) { *aborted = 1u; break; }
                tc_fence_after();
                uint8_t* st = smem + (size_t)s * Cfg::STAGE_BYTES;
                const uint64_t db = smem_desc_sw128(st + Cfg::A_BYTES);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {   // accumulator (mt, nb) lives at TMEM column (mt * NB + nb) * BN
                    const uint64_t da = smem_desc_sw128(st + mt * GM_BM * GM_BK * 2);
#pragma unroll
                    for (int k = 0; k < GM_BK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        umma_bf16(tmem_base + mt * Cfg::NB * BN, da + 2 * k, db + 2 * k, idesc, acc);   // +32 bytes per K=16 step
                    }
                }
                umma_commit(&empty[s]);     // frees this stage once the MMAs above have read it
            }
            umma_commit(accum);             // accumulator complete (or, after an expired wait, the MMAs issued so far)
            if (*aborted) mbar_wait_drain(accum, 0);   // tensor memory is freed below: nothing may still be writing it
        }
        __syncwarp();
    } else {
        // epilogue: warp (2..9) owns TMEM lanes 32*(warp%4) .. +31 = tile rows and half of the columns
        const bool acc_ok = mbar_wait(accum, 0, status) && !*aborted;   // after an expired wait nothing is read or stored
        tc_fence_after();
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        // the two warps of a quarter take one 128-row accumulator each (MT = 2) or half of the columns (MT = 1)
        static_assert(GM_EPI_WARPS == 8 && (MT == 2 || (BN / 2) % 32 == 0), "epilogue split");
        const int cbeg = MT == 2 ? 0 : half * (BN / 2), cend = MT == 2 ? BN : cbeg + BN / 2;
#pragma unroll 1
        for (int mt = (MT == 2 ? half : 0); mt < (MT == 2 ? half + 1 : 1); ++mt) {
        if (!acc_ok) break;
        const int row = m0 + mt * GM_BM + quarter * 32 + lane;
        const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * Cfg::NB * BN);
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(trow + c0, v);
            if (EPI == EPI_PARTIAL) {   // raw fp32 accumulators into plane blockIdx.z of C (a float [gridDim.z][M][ldc] array)
                if (row < M) {
                    float4* fp = reinterpret_cast<float4*>(reinterpret_cast<float*>(C) + ((size_t)blockIdx.z * M + row) * ldc + n0 + c0);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        fp[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                }
                continue;
            }
            uint32_t out[16];
            if (EPI == EPI_SWIGLU) {
                uint32_t u[32];
                tmem_ld32(trow + BN + c0, u);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float g0 = rbf(__uint_as_float(v[2 * j])), g1 = rbf(__uint_as_float(v[2 * j + 1]));
                    const float u0 = rbf(__uint_as_float(u[2 * j])), u1 = rbf(__uint_as_float(u[2 * j + 1]));
                    out[j] = pack_bf16x2(rbf(silu_fast(g0)) * u0, rbf(silu_fast(g1)) * u1);
                }
            } else if (EPI == EPI_RESID) {
                if (row < M) {
                    const uint4* rp = reinterpret_cast<const uint4*>(R + (size_t)row * ldc + n0 + c0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 rr = rp[q];
                        const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = q * 4 + e;
                            out[j] = pack_bf16x2(bf_lo(rw[e]) + rbf(__uint_as_float(v[2 * j])), bf_hi(rw[e]) + rbf(__uint_as_float(v[2 * j + 1])));
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) out[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            }
            if (row < M) {
                uint4* cp = reinterpret_cast<uint4*>(C + (size_t)row * ldc + n0 + c0);
#pragma unroll
                for (int q = 0; q < 4; ++q) cp[q] = make_uint4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
            }
        }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (*aborted) {
        // After an expired wait (anybody's: the flag is read behind the barrier): copies that were requested still
        // land in this CTA's shared memory, so the producer waits for the last one of every stage before the CTA exits.
        if (tid == 0)
            for (int s = 0; s < Cfg::STAGES && s < issued; ++s) {
                const int last = ((issued - 1 - s) / Cfg::STAGES) * Cfg::STAGES + s;      // last requested k-block of stage s
                if (last != drop_kb) mbar_wait_drain(&full[s], (uint32_t)(last / Cfg::STAGES) & 1u);
            }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---------------------------------------------------------------- skinny GEMM for M <= 64 (batched decode)
// With a handful of activation rows the linears are weight-streaming problems: a
// 128-row output tile per CTA gives 8-48 CTAs, each latency-bound on its own TMA
// ring.  Here the operands are swapped (the 128 weight rows of a tile are the MMA's
// M dimension, the batch is its N) and K is split across CTAs, so every GEMM
// spreads over roughly all SMs and each CTA has its whole K slice in flight at
// once.  Each CTA writes an fp32 partial tile part[ks][b][n]; the consumer kernels
// below sum the K splits in a fixed order (deterministic) and apply the bf16
// rounding, residual, norm or SwiGLU.
constexpr int SK_MAXKB = 6;       // k-blocks (64 columns) per CTA, all in flight

template <int MPAD>
__global__ void __launch_bounds__(GM_THREADS, 1)
k_gemm_skinny(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmW2,
              int tiles0, int tiles1, const __grid_constant__ CUtensorMap tmX, float* __restrict__ part, int M, int ldp,
              int kb_per_cta, unsigned int* status) {
    pdl_trigger();   // the next grid may be scheduled already
    // The weight tiles do not depend on the preceding kernel: they are requested before
    // griddepcontrol.wait and arrive while that kernel is still running; only the activation
    // tiles (and everything downstream of them) come after the wait.
    // Up to three weight matrices are concatenated along the output dimension (q|k|v,
    // gate|up): tile blockIdx.x belongs to matrix 0, 1 or 2; ldp is the row length of
    // one partial plane part[ks] = [M, ldp].
    constexpr int W_BYTES = 128 * GM_BK * 2, X_BYTES = MPAD * GM_BK * 2;
    constexpr int TM_COLS = MPAD < 32 ? 32 : MPAD;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // the launch sizes the dynamic shared memory for kb_per_cta k-blocks (not the maximum), so that CTAs with short K
    // slices fit two to an SM and a grid of up to 2 x SMs CTAs runs in one round
    uint8_t* xs = smem + kb_per_cta * W_BYTES;                             // X tiles, each 1024-byte aligned
    constexpr int X_STRIDE = (X_BYTES + 1023) & ~1023;
    uint64_t* full = reinterpret_cast<uint64_t*>(xs + kb_per_cta * X_STRIDE);
    uint64_t* accum = full + SK_MAXKB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x, ks = blockIdx.y;
    const int kb0 = ks * kb_per_cta;
    const CUtensorMap* tmW = tile < tiles0 ? &tmW0 : (tile < tiles0 + tiles1 ? &tmW1 : &tmW2);
    const int wrow0 = (tile < tiles0 ? tile : (tile < tiles0 + tiles1 ? tile - tiles0 : tile - tiles0 - tiles1)) * 128;

    if (tid == 0) {
        for (int s = 0; s < SK_MAXKB; ++s) mbar_init(&full[s], 1);
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < kb_per_cta; ++i) {
                mbar_expect_tx(&full[i], (uint32_t)(W_BYTES + X_BYTES));
                tma_load_2d(smem + i * W_BYTES, tmW, (kb0 + i) * GM_BK, wrow0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < kb_per_cta; ++i) tma_load_2d(xs + i * X_STRIDE, &tmX, (kb0 + i) * GM_BK, 0, &full[i]);
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MPAD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            for (int i = 0; i < kb_per_cta; ++i) {
                mbar_wait(&full[i], 0, status);
                tc_fence_after();
                const uint64_t dw = smem_desc_sw128(smem + i * W_BYTES);
                const uint64_t dx = smem_desc_sw128(xs + i * X_STRIDE);
#pragma unroll
                for (int k = 0; k < GM_BK / 16; ++k) umma_bf16(tmem_base, dw + 2 * k, dx + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(accum);
        }
        __syncwarp();
    } else {
        mbar_wait(accum, 0, status);
        tc_fence_after();
        const int quarter = warp & 3;
        const int n = tile * 128 + quarter * 32 + lane;
        const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float* dst = part + (size_t)ks * M * ldp + n;
#pragma unroll
        for (int c0 = 0; c0 < MPAD; c0 += 16) {
            uint32_t v[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                : "r"(trow + c0) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (c0 + j < M) dst[(size_t)(c0 + j) * ldp] = __uint_as_float(v[j]);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TM_COLS);
}

// consumers of the fp32 K-split partials part[ks][row][col] (ks summed in index order)
template <int KS>
__device__ __forceinline__ float sum_planes(const float* part, size_t plane, size_t idx) {
    float v[KS];
#pragma unroll
    for (int k = 0; k < KS; ++k) v[k] = part[(size_t)k * plane + idx];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) s += v[k];
    return s;
}
__device__ __forceinline__ float sum_splits(const float* part, int ksplit, size_t plane, size_t idx) {
    // every plane is requested before the first is used (a loop of unknown length would wait for one L2 round trip
    // per plane); the sum runs in plane order whatever the count, so the result does not depend on this dispatch
    switch (ksplit) {
    case 2: return sum_planes<2>(part, plane, idx);
    case 4: return sum_planes<4>(part, plane, idx);
    case 8: return sum_planes<8>(part, plane, idx);
    default: break;
    }
    float s = 0.f;
    for (int k = 0; k < ksplit; ++k) s += part[(size_t)k * plane + idx];
    return s;
}
template <int KS>
__device__ __forceinline__ float4 sum_planes4(const float* part, size_t plane, size_t idx) {
    float4 v[KS];
#pragma unroll
    for (int k = 0; k < KS; ++k) v[k] = *reinterpret_cast<const float4*>(part + (size_t)k * plane + idx);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < KS; ++k) { a.x += v[k].x; a.y += v[k].y; a.z += v[k].z; a.w += v[k].w; }
    return a;
}


// h = bf16(h + bf16(sum));  x = rmsnorm(h) * w      one CTA per row (N = 1024), 4 columns per thread
__global__ void __launch_bounds__(256) k_sk_resid_norm(const float* __restrict__ part, int ksplit, int M, bf16* __restrict__ h,
                                                       const bf16* __restrict__ w, bf16* __restrict__ x) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    __shared__ float s_red[8];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t base = (size_t)row * H + 4 * tid, plane = (size_t)M * H;
    const uint2 hu = *reinterpret_cast<const uint2*>(h + base);
    const uint2 wu = w ? *reinterpret_cast<const uint2*>(w + 4 * tid) : make_uint2(0u, 0u);   // requested with the planes, used after the row sum
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ksplit == 8) acc = sum_planes4<8>(part, plane, base);
    else if (ksplit == 2) acc = sum_planes4<2>(part, plane, base);
    else if (ksplit == 4) acc = sum_planes4<4>(part, plane, base);
    else
        for (int k = 0; k < ksplit; ++k) {
            const float4 p = *reinterpret_cast<const float4*>(part + (size_t)k * plane + base);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
    float v[4] = {rbf(bf_lo(hu.x) + rbf(acc.x)), rbf(bf_hi(hu.x) + rbf(acc.y)), rbf(bf_lo(hu.y) + rbf(acc.z)), rbf(bf_hi(hu.y) + rbf(acc.w))};
    *reinterpret_cast<uint2*>(h + base) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    if (!w) return;   // residual stream only (after the last layer nothing is normalised here)
    float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_red[i];
    const float r = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
    const uint2 o = make_uint2(pack_bf16x2(rbf(bf_lo(wu.x) * rbf(v[0] * r)), rbf(bf_hi(wu.x) * rbf(v[1] * r))),
                               pack_bf16x2(rbf(bf_lo(wu.y) * rbf(v[2] * r)), rbf(bf_hi(wu.y) * rbf(v[3] * r))));
    *reinterpret_cast<uint2*>(x + base) = o;
}

// act[row, c] = bf16( bf16(silu(bf16(sum gate))) * bf16(sum up) )   gate/up partials are column blocks [0,I) and [I,2I)
__global__ void __launch_bounds__(256) k_sk_swiglu(const float* __restrict__ part, int ksplit, int M, bf16* __restrict__ act) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (size_t)M * I) return;
    const int row = (int)(i / I), col = (int)(i % I);
    const size_t plane = (size_t)M * 2 * I, base = (size_t)row * 2 * I + col;
    const float g = rbf(sum_splits(part, ksplit, plane, base)), u = rbf(sum_splits(part, ksplit, plane, base + I));
    act[i] = __float2bfloat16_rn(rbf(silu_f32(g)) * u);
}

// ---------------------------------------------------------------- row-wise kernels
// h[s,:] = embed[ids[s],:]      (reference: prefill_embed_kernel, fused_prefill_kernels.inl:3-20)
// Rows audio_start .. audio_start + audio_len - 1 take externally computed embeddings instead
// (reference: prefill_patch_audio_kernel, fused_prefill_kernels.inl:28-45, a separate launch there).
__global__ void __launch_bounds__(128) k_pf_embed(const int* __restrict__ ids, const bf16* __restrict__ embed, bf16* __restrict__ h,
                                                  int vocab, unsigned int* status, const bf16* __restrict__ audio = nullptr,
                                                  int audio_start = 0, int audio_len = 0) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    const int s = blockIdx.x;
    if (audio != nullptr && s >= audio_start && s < audio_start + audio_len) {
        reinterpret_cast<uint4*>(h + (size_t)s * H)[threadIdx.x] =
            __ldg(reinterpret_cast<const uint4*>(audio + (size_t)(s - audio_start) * H) + threadIdx.x);
        return;
    }
    int tok = ids[s];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, MQ_STATUS_BAD_TOKEN);
        tok = min(max(tok, 0), vocab - 1);
    }
    reinterpret_cast<uint4*>(h + (size_t)s * H)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(embed + (size_t)tok * H) + threadIdx.x);
}

// x[s,:] = bf16( w * bf16( h[s,:] * rsqrt(mean(h^2) + eps) ) )   one warp per row
// (reference: prefill_rmsnorm_kernel, fused_prefill_kernels.inl:52-105)
__global__ void __launch_bounds__(256) k_pf_rmsnorm(const bf16* __restrict__ h, const bf16* __restrict__ w, bf16* __restrict__ x, int rows) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float v[32];
    const bf16* src = h + (size_t)row * H;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 u = *reinterpret_cast<const uint4*>(src + j * 256 + lane * 8);
        v[j * 8 + 0] = bf_lo(u.x); v[j * 8 + 1] = bf_hi(u.x); v[j * 8 + 2] = bf_lo(u.y); v[j * 8 + 3] = bf_hi(u.y);
        v[j * 8 + 4] = bf_lo(u.z); v[j * 8 + 5] = bf_hi(u.z); v[j * 8 + 6] = bf_lo(u.w); v[j * 8 + 7] = bf_hi(u.w);
    }
    rmsnorm_slice(v, w, lane);
    bf16* dst = x + (size_t)row * H;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint4 o;
        o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]); o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
        o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]); o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
        *reinterpret_cast<uint4*>(dst + j * 256 + lane * 8) = o;
    }
}

// Per (position, head): q/k heads get RMSNorm(128) * w and split-half RoPE evaluated in
// bf16; q stays in the qkv buffer, k and v go to the cache at position pos0 + s
// (reference: prefill_qk_norm_rope_kernel, fused_prefill_kernels.inl:112-258).
// One warp per head: 16 q + 8 k + 8 v = 32 warps per position.
__global__ void __launch_bounds__(256) k_pf_qknorm_rope(bf16* __restrict__ qkv, const bf16* __restrict__ wq, const bf16* __restrict__ wk,
                                                        const bf16* __restrict__ cos, const bf16* __restrict__ sin, bf16* __restrict__ k_cache,
                                                        bf16* __restrict__ v_cache, int layer, int pos0, int max_seq,
                                                        const int* __restrict__ pos_rows, size_t seq_stride,
                                                        const float* __restrict__ part, int ksplit, int M,
                                                        const int* __restrict__ row_seq) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    // pos_rows == nullptr: one sequence, row s sits at position pos0 + s.
    // pos_rows != nullptr: row s is at position pos_rows[s] of sequence row_seq[s] (sequence s if row_seq is
    // null), whose cache starts that many times seq_stride elements in.
    // part != nullptr: the raw q|k|v row is not in qkv yet but in ksplit fp32 partial planes part[ks][M][QKV]
    // of a K-split GEMM; they are summed in index order and rounded to bf16 here (q is then written to qkv).
    // A warp handles units (q heads 0..15, k heads 16..23, v heads 24..31) blockIdx.y * 8 + warp,
    // then every gridDim.y * 8 further: one CTA per row with gridDim.y = 1, four with 4.
    const int lane = threadIdx.x & 31;
    const int s = blockIdx.x;
    const int pos = pos_rows ? min(max(pos_rows[s], 0), max_seq - 1) : pos0 + s;
    if (pos_rows) {
        const size_t seq = row_seq ? (size_t)row_seq[s] : (size_t)s;
        k_cache += seq * seq_stride;
        v_cache += seq * seq_stride;
    }
    bf16* row = qkv + (size_t)s * QKV;
    const bf16* cosr = cos + (size_t)pos * D;
    const bf16* sinr = sin + (size_t)pos * D;
    const uint32_t cl = *reinterpret_cast<const uint32_t*>(cosr + 2 * lane), chh = *reinterpret_cast<const uint32_t*>(cosr + 64 + 2 * lane);
    const uint32_t sl = *reinterpret_cast<const uint32_t*>(sinr + 2 * lane), sh = *reinterpret_cast<const uint32_t*>(sinr + 64 + 2 * lane);
    const float clo[2] = {bf_lo(cl), bf_hi(cl)}, chi[2] = {bf_lo(chh), bf_hi(chh)};
    const float slo[2] = {bf_lo(sl), bf_hi(sl)}, shi[2] = {bf_lo(sh), bf_hi(sh)};
    for (int unit = blockIdx.y * 8 + (threadIdx.x >> 5); unit < NQ + 2 * NKV; unit += gridDim.y * 8) {
        if (unit >= NQ + NKV) {   // V head: raw copy into the cache
            const int g = unit - NQ - NKV;
            uint2 u;
            if (part) {
                const size_t i0 = (size_t)s * QKV + QSZ + KVSZ + g * D + 4 * lane;
                float f[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) f[e] = sum_splits(part, ksplit, (size_t)M * QKV, i0 + e);
                u = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
            } else {
                u = *reinterpret_cast<const uint2*>(row + QSZ + KVSZ + g * D + 4 * lane);
            }
            *reinterpret_cast<uint2*>(v_cache + ((size_t)(layer * NKV + g) * max_seq + pos) * D + 4 * lane) = u;
            continue;
        }
        const bool is_q = unit < NQ;
        bf16* head = is_q ? row + unit * D : row + QSZ + (unit - NQ) * D;
        const bf16* wn = is_q ? wq : wk;
        float xl[2], xh[2];
        if (part) {
            const size_t i0 = (size_t)s * QKV + (size_t)(head - row) + 2 * lane;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                xl[e] = rbf(sum_splits(part, ksplit, (size_t)M * QKV, i0 + e));
                xh[e] = rbf(sum_splits(part, ksplit, (size_t)M * QKV, i0 + 64 + e));
            }
        } else {
            const uint32_t ulo = *reinterpret_cast<const uint32_t*>(head + 2 * lane), uhi = *reinterpret_cast<const uint32_t*>(head + 64 + 2 * lane);
            xl[0] = bf_lo(ulo); xl[1] = bf_hi(ulo); xh[0] = bf_lo(uhi); xh[1] = bf_hi(uhi);
        }
        const uint32_t wl = *reinterpret_cast<const uint32_t*>(wn + 2 * lane), wh = *reinterpret_cast<const uint32_t*>(wn + 64 + 2 * lane);
        float ss = xl[0] * xl[0] + xl[1] * xl[1] + xh[0] * xh[0] + xh[1] * xh[1];
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
        const float wlo[2] = {bf_lo(wl), bf_hi(wl)}, whi[2] = {bf_lo(wh), bf_hi(wh)};
        float lo[2], hi[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float nl = rbf(wlo[e] * rbf(xl[e] * r));
            const float nh = rbf(whi[e] * rbf(xh[e] * r));
            lo[e] = rbf(rbf(nl * clo[e]) + rbf(-nh * slo[e]));
            hi[e] = rbf(rbf(nh * chi[e]) + rbf(nl * shi[e]));
        }
        const uint32_t plo = pack_bf16x2(lo[0], lo[1]), phi = pack_bf16x2(hi[0], hi[1]);
        bf16* dst = is_q ? head : k_cache + ((size_t)(layer * NKV + (unit - NQ)) * max_seq + pos) * D;
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = phi;
    }
}

// ---------------------------------------------------------------- causal GQA attention (prefill)
// QK^T and PV run on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with an online softmax in
// registers; probabilities are rounded to bf16 before the PV product and the row sum uses the
// unrounded values.
// Causal attention of the prompt.  One CTA per (query head, 64-query tile).  Under the causal
// mask the last query tile of a prompt has sixteen times the work of the first, and the pass
// is as long as its longest CTA, so the key tiles of a query tile are dealt out to FA_NG
// groups of four warps that walk them in parallel (group g takes key tiles g, g + FA_NG, ..)
// and are merged through shared memory at the end; the grid is ordered longest query tile
// first.  Each group streams its K/V tiles through its own two-stage ring of padded rows
// (16-byte cp.async, the next tile in flight while this one is multiplied).
constexpr int FA_BQ = 64, FA_BK = 64, FA_LD = D + 8, FA_NG = 2, FA_THREADS = FA_NG * 128;
constexpr int FA_TILE_ELEMS = FA_BK * FA_LD;                                  // one K or V tile
struct PackedTiles {          // all null / zero for a single prompt
    const int* tile_seq;      // [tiles] sequence of query tile t
    const int* tile_q0;       // [tiles] first query row of the tile inside its sequence
    const int* seq_len;       // [sequences]
    const int* seq_row0;      // [sequences] first packed row of the sequence
    size_t seq_stride;        // elements between the caches of consecutive sequences
};
constexpr size_t FA_SMEM = (size_t)(FA_BQ * FA_LD + FA_NG * 2 * 2 * FA_TILE_ELEMS) * 2;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t n = valid ? 16u : 0u;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(FA_THREADS, 1) k_pf_attention(const bf16* __restrict__ qkv, const bf16* __restrict__ k_cache,
                                                               const bf16* __restrict__ v_cache, bf16* __restrict__ out, int S, int pos0,
                                                               int layer, int max_seq, PackedTiles pt) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    extern __shared__ __align__(16) uint8_t fa_smem[];
    bf16* sq = reinterpret_cast<bf16*>(fa_smem);                    // [64][FA_LD]
    bf16* ring = sq + FA_BQ * FA_LD;                                // [FA_NG][2 stages][K tile | V tile]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = warp >> 2, wq = warp & 3, gtid = tid & 127;
    const int head = blockIdx.x, g = head / (NQ / NKV);
    int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * FA_BQ;  // longest query tiles are dispatched first
    if (pt.tile_seq) {   // several prompts packed row after row: tile blockIdx.y belongs to one of them (the host sorts long tiles first)
        const int b = pt.tile_seq[blockIdx.y];
        q0 = pt.tile_q0[blockIdx.y];
        S = pt.seq_len[b];
        const size_t row0 = (size_t)pt.seq_row0[b];
        qkv += row0 * QKV;
        out += row0 * QSZ;
        k_cache += (size_t)b * pt.seq_stride;
        v_cache += (size_t)b * pt.seq_stride;
    }
    const bf16* kbase = k_cache + ((size_t)(layer * NKV + g) * max_seq) * D;
    const bf16* vbase = v_cache + ((size_t)(layer * NKV + g) * max_seq) * D;
    bf16* gring = ring + (size_t)grp * 4 * FA_TILE_ELEMS;

    const int kv_end = min(pos0 + S, pos0 + q0 + FA_BQ);     // exclusive bound of keys any row of the tile may see
    const int ntiles = (kv_end + FA_BK - 1) / FA_BK;
    auto load_tile = [&](int t, int stage) {
        bf16* sk = gring + (size_t)stage * 2 * FA_TILE_ELEMS;
        bf16* sv = sk + FA_TILE_ELEMS;
        const int p0 = t * FA_BK;
        for (int c = gtid; c < FA_BK * (D / 8); c += 128) {
            const int r = c / (D / 8), cc = c % (D / 8);
            const bool ok = p0 + r < kv_end;
            const size_t off = (size_t)(ok ? p0 + r : 0) * D + cc * 8;
            cp_async16_zfill(sk + r * FA_LD + cc * 8, kbase + off, ok);
            cp_async16_zfill(sv + r * FA_LD + cc * 8, vbase + off, ok);
        }
    };
    if (grp < ntiles) load_tile(grp, 0);
    cp_async_commit();

    // Q tile -> shared (rows past S are zero)
    for (int c = tid; c < FA_BQ * (D / 8); c += FA_THREADS) {
        const int r = c / (D / 8), cc = c % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (q0 + r < S) v = *reinterpret_cast<const uint4*>(qkv + (size_t)(q0 + r) * QKV + head * D + cc * 8);
        *reinterpret_cast<uint4*>(sq + r * FA_LD + cc * 8) = v;
    }
    __syncthreads();
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
        ldsm_x4(qf[kk], sq + (wq * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * FA_LD + kk * 16 + (lane >> 4) * 8);

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
    // scores are kept in the log2 domain (scale * log2(e) folded in) so that the softmax uses
    // the single-instruction exp2 instead of expf; the probabilities are the same numbers
    const float scale = 0.08838834764831845f * 1.4426950408889634f;
    const int row_a = pos0 + q0 + wq * 16 + (lane >> 2);   // absolute position of this thread's first row; second is +8

    int it = 0;
    for (int t = grp; t < ntiles; t += FA_NG, ++it) {
        // the other stage was consumed in the previous iteration (barrier at its end): request the next tile
        if (t + FA_NG < ntiles) load_tile(t + FA_NG, (it + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();          // this thread's copies of tile t have landed
        group_barrier(grp);          // .. and everybody's in the group
        const bf16* sk = gring + (size_t)(it & 1) * 2 * FA_TILE_ELEMS;
        const bf16* sv = sk + FA_TILE_ELEMS;
        const int p0 = t * FA_BK;

        float sacc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {   // pairs of 8-key tiles
                uint32_t kf[4];
                ldsm_x4(kf, sk + (np * 16 + (lane & 7) + (lane >> 4) * 8) * FA_LD + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(sacc[2 * np], qf[kk], kf[0], kf[1]);
                mma_bf16_16816(sacc[2 * np + 1], qf[kk], kf[2], kf[3]);
            }
        }
        // scale, causal mask, online softmax
        float mx[2] = {-1e30f, -1e30f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = p0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                const int rowp = row_a + (e >> 1) * 8;
                const float sv_ = (key <= rowp) ? sacc[nt][e] * scale : -1e30f;
                sacc[nt][e] = sv_;
                mx[e >> 1] = fmaxf(mx[e >> 1], sv_);
            }
        }
        float corr[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
            const float m_new = fmaxf(m_run[h2], mx[h2]);
            corr[h2] = fast_exp2(m_run[h2] - m_new);
            m_run[h2] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pf[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float pe[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pe[e] = (sacc[nt][e] <= -1e29f) ? 0.f : fast_exp2(sacc[nt][e] - m_run[e >> 1]);
                rs[e >> 1] += pe[e];
            }
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(pe[0], pe[1]);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(pe[2], pe[3]);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            rs[h2] += __shfl_xor_sync(0xffffffffu, rs[h2], 1);
            rs[h2] += __shfl_xor_sync(0xffffffffu, rs[h2], 2);
            l_run[h2] = l_run[h2] * corr[h2] + rs[h2];
        }
#pragma unroll
        for (int dt = 0; dt < 16; ++dt) { o[dt][0] *= corr[0]; o[dt][1] *= corr[0]; o[dt][2] *= corr[1]; o[dt][3] *= corr[1]; }
        // O += P V
#pragma unroll
        for (int j = 0; j < 4; ++j) {          // 16 keys per step
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {   // pairs of 8-wide output tiles
                uint32_t vf[4];
                ldsm_x4_t(vf, sv + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * FA_LD + dp * 16 + (lane >> 4) * 8);
                mma_bf16_16816(o[2 * dp], pf[j], vf[0], vf[1]);
                mma_bf16_16816(o[2 * dp + 1], pf[j], vf[2], vf[3]);
            }
        }
        group_barrier(grp);          // the stage may be overwritten by the next iteration's request
    }
    cp_async_wait_all();
    __syncthreads();
    // merge the groups: groups 1.. leave (m, l, O) of every thread in the ring, group 0 combines
    float* xch = reinterpret_cast<float*>(ring);        // [FA_NG - 1][128 threads][68]
    if (grp > 0) {
        float* mine = xch + ((size_t)(grp - 1) * 128 + gtid) * 68;
        mine[0] = m_run[0]; mine[1] = m_run[1]; mine[2] = l_run[0]; mine[3] = l_run[1];
#pragma unroll
        for (int dt = 0; dt < 16; ++dt) *reinterpret_cast<float4*>(mine + 4 + dt * 4) = make_float4(o[dt][0], o[dt][1], o[dt][2], o[dt][3]);
    }
    __syncthreads();
    if (grp > 0) return;
#pragma unroll
    for (int og = 1; og < FA_NG; ++og) {
        const float* oth = xch + ((size_t)(og - 1) * 128 + gtid) * 68;
        float f_me[2], f_ot[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const float mo = oth[h2], mn = fmaxf(m_run[h2], mo);
            f_me[h2] = fast_exp2(m_run[h2] - mn);
            f_ot[h2] = fast_exp2(mo - mn);
            l_run[h2] = l_run[h2] * f_me[h2] + oth[2 + h2] * f_ot[h2];
            m_run[h2] = mn;
        }
#pragma unroll
        for (int dt = 0; dt < 16; ++dt) {
            const float4 ov = *reinterpret_cast<const float4*>(oth + 4 + dt * 4);
            o[dt][0] = o[dt][0] * f_me[0] + ov.x * f_ot[0];
            o[dt][1] = o[dt][1] * f_me[0] + ov.y * f_ot[0];
            o[dt][2] = o[dt][2] * f_me[1] + ov.z * f_ot[1];
            o[dt][3] = o[dt][3] * f_me[1] + ov.w * f_ot[1];
        }
    }
    // normalise and store
    const int r_lo = q0 + wq * 16 + (lane >> 2), r_hi = r_lo + 8;
    const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[1];
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) {
        const int col = head * D + dt * 8 + (lane & 3) * 2;
        if (r_lo < S) *reinterpret_cast<uint32_t*>(out + (size_t)r_lo * QSZ + col) = pack_bf16x2(o[dt][0] * inv0, o[dt][1] * inv0);
        if (r_hi < S) *reinterpret_cast<uint32_t*>(out + (size_t)r_hi * QSZ + col) = pack_bf16x2(o[dt][2] * inv1, o[dt][3] * inv1);
    }
}

// ---------------------------------------------------------------- causal attention on tcgen05 (one prompt)
// One CTA per (query head, 128-query tile); key tiles of 128 positions.  Both contractions run
// on the 5th-generation tensor cores with their accumulators in tensor memory:
//     S = Q K^T     A = Q tile [128 q x 128 d], B = K tile [128 keys x 128 d] straight from the KV cache
//     O_j = P V     A = P tile [128 q x 128 keys] (bf16) IN TENSOR MEMORY: the softmax warps write the probabilities
//                   over the scores they came from (tcgen05.st; 64 packed columns of S's 128), so the product
//                   reads only V from shared memory and nothing crosses the generic / async proxy boundary,
//                   B = V tile [128 keys x 128 d] straight from the KV cache, read as an MN-major operand
//                   (the cache rows are contiguous along d, the product contracts over the keys)
// (128-byte swizzle, fetched by TMA; the V map ends at the last key of the prompt, so the rows of the
// last tile beyond it arrive as zeros whatever the cache holds there).  Warp 0 feeds the K / V
// rings, warp 1 issues the MMAs, warps 2-9 hold HALF A QUERY ROW PER THREAD: they read the row's
// scores from tensor memory (tcgen05.ld), keep the running max / sum and write the probabilities
// rounded to bf16 as the next MMA's A operand; the output accumulates in tensor memory and is
// rescaled (tcgen05.ld / st) only when the maximum has grown by more than 2^8.  S is
// double-buffered: QK^T of tile j + 1 runs while tile j is in the softmax.  Replaces the reference's serial-per-warp kernel and its experimental tiles
// (csrc/megakernel/fused_prefill_kernels.inl:265-342, 347-445, 486-613).
constexpr int TA_BQ = 128, TA_BK = 128;
constexpr int TA_THREADS = 320;                             // warp 0 TMA, warp 1 MMA, warps 2-9 softmax
constexpr int TA_TILE_BYTES = 128 * 128 * 2;               // two 64-column halves of [128 rows x 128 bytes]
constexpr int TA_HALF_BYTES = TA_TILE_BYTES / 2;
constexpr size_t TA_SMEM = (size_t)5 * TA_TILE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + TA_BQ * 8 /*row exchange*/;   // Q, 2 K, 2 V
static_assert(TA_SMEM <= 232448, "shared memory of one CTA");
constexpr uint32_t TA_TMEM_COLS = 512;                      // S0 | S1 | O (128 columns each)


__global__ void __launch_bounds__(TA_THREADS, 1)
k_pf_attention_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  bf16* __restrict__ out, int S, int pos0, int layer, int max_seq, unsigned int* status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ uint8_t ta_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ta_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TA_TILE_BYTES;            // [2]
    uint8_t* sV = sK + 2 * TA_TILE_BYTES;        // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * TA_TILE_BYTES);
    uint64_t* q_full = bars;                     // 1
    uint64_t* k_full = bars + 1;                 // 2
    uint64_t* k_empty = bars + 3;                // 2
    uint64_t* v_full = bars + 5;                 // 2
    uint64_t* v_empty = bars + 7;                // 2
    uint64_t* s_full = bars + 9;                 // 2
    uint64_t* s_free = bars + 11;                // 2 (256 arrivals)
    uint64_t* p_full = bars + 13;                // 2 (256 arrivals)
    uint64_t* o_full = bars + 17;                // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
    float (*xm)[2] = reinterpret_cast<float(*)[2]>(bars + 20);   // [128][2]: the two half-row maxima (at the end: sums) of a query row

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.x, g = head / (NQ / NKV);
    const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * TA_BQ;        // longest query tiles first
    const int kv_end = min(pos0 + S, pos0 + q0 + TA_BQ);                  // keys any row of the tile may see
    const int nt = (kv_end + TA_BK - 1) / TA_BK;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 256); mbar_init(&p_full[i], 256);
        }
        mbar_init(o_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TA_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t tmem_o = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, TA_TILE_BYTES);
            tma_load_2d(sQ, &tmQ, head * D, q0, q_full);
            tma_load_2d(sQ + TA_HALF_BYTES, &tmQ, head * D + 64, q0, q_full);
            const int krow0 = (layer * NKV + g) * max_seq;
            for (int j = 0; j < nt; ++j) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&k_empty[st], (uint32_t)((j >> 1) - 1) & 1u, status)) break;
                mbar_expect_tx(&k_full[st], TA_TILE_BYTES);
                tma_load_2d(sK + st * TA_TILE_BYTES, &tmK, 0, krow0 + j * TA_BK, &k_full[st]);
                tma_load_2d(sK + st * TA_TILE_BYTES + TA_HALF_BYTES, &tmK, 64, krow0 + j * TA_BK, &k_full[st]);
                if (j >= 2 && !mbar_wait(&v_empty[st], (uint32_t)((j >> 1) - 1) & 1u, status)) break;
                mbar_expect_tx(&v_full[st], TA_TILE_BYTES);
                tma_load_3d(sV + st * TA_TILE_BYTES, &tmV, 0, j * TA_BK, layer * NKV + g, &v_full[st]);
                tma_load_3d(sV + st * TA_TILE_BYTES + TA_HALF_BYTES, &tmV, 64, j * TA_BK, layer * NKV + g, &v_full[st]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint32_t idesc_pv = idesc | (1u << 16);    // B (the V tile) is MN-major
            bool ok = mbar_wait(q_full, 0, status);
            auto issue_s = [&](int j) {      // S[j & 1] = Q K_j^T
                const int st = j & 1;
                ok = ok && mbar_wait(&k_full[st], (uint32_t)(j >> 1) & 1u, status);
                if (j >= 2) ok = ok && mbar_wait(&s_free[st], (uint32_t)((j >> 1) - 1) & 1u, status);
                tc_fence_after();
                if (ok) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint64_t da = smem_desc_sw128(sQ + (kk >> 2) * TA_HALF_BYTES) + 2 * (kk & 3);
                        const uint64_t db = smem_desc_sw128(sK + st * TA_TILE_BYTES + (kk >> 2) * TA_HALF_BYTES) + 2 * (kk & 3);
                        umma_bf16(tmem_base + st * 128, da, db, idesc, kk > 0 ? 1u : 0u);
                    }
                }
                umma_commit(&k_empty[st]);
                umma_commit(&s_full[st]);
            };
            issue_s(0);
            for (int j = 0; j < nt; ++j) {
                const int st = j & 1;
                if (j + 1 < nt) issue_s(j + 1);
                ok = ok && mbar_wait(&p_full[st], (uint32_t)(j >> 1) & 1u, status);
                ok = ok && mbar_wait(&v_full[st], (uint32_t)(j >> 1) & 1u, status);
                tc_fence_after();
                if (ok) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        // A = the probabilities, written by the softmax threads over the scores they came from: 16 keys
                        // of a row are eight 32-bit columns.  B: 16 keys per step = two 1024-byte groups of the
                        // [keys][64 d] panels (d 0-63 | d 64-127)
                        const uint64_t db = smem_desc_mn_sw128(sV + st * TA_TILE_BYTES, TA_HALF_BYTES) + (uint64_t)(kk * (2048 >> 4));
                        umma_bf16_ts(tmem_o, tmem_base + st * 128 + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);   // O accumulates over all key tiles
                    }
                }
                umma_commit(&v_empty[st]);
                umma_commit(o_full);
            }
        }
        __syncwarp();
    } else {
        // softmax warps: TWO threads per query row r = TMEM lane r (warps w and w + 4 share a quarter of the
        // lanes); thread `half` owns keys [64 half, 64 half + 64) of every key tile and output columns
        // [64 half, +64).  The two exchange their half-row maxima through shared memory (one 64-thread
        // named barrier per tile), so both scale by the same running maximum.  The output accumulates in
        // tensor memory over all key tiles; it is only rescaled when the running maximum has grown by
        // more than 2^8 since the value the accumulator is scaled to (then p <= 256 in between, exact in
        // fp32 and harmless in bf16), which after the first tiles practically never happens.  With one
        // thread per row the 128 exponentials per tile on four warps (one per scheduler) bounded the kernel.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const uint32_t col_off = (uint32_t)(half * 64);
        const int qpos = pos0 + q0 + r;                       // absolute position of this thread's query
        const float c = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
        float m = -INFINITY, l = 0.f;                         // m: the maximum the sums are scaled to (raw score units)
        bool ok = true;
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
        for (int j = 0; j < nt; ++j) {
            const int st = j & 1;
            const uint32_t ts = tmem_base + st * 128 + lane_off + col_off;
            ok = ok && mbar_wait(&s_full[st], (uint32_t)(j >> 1) & 1u, status);
            tc_fence_after();
            const int k0 = j * TA_BK + half * 64;             // first key of this thread's half
            const bool diag = k0 + 63 > qpos;                 // some keys of this half lie beyond the query
            uint32_t sv[64];
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) tmem_ld32_nowait(ts + cb * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[cb * 32]));
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&s_free[st]);                         // the scores are in registers: S[st] may be overwritten
            float mh = -INFINITY;
            if (__any_sync(0xffffffffu, diag)) {              // only the last one or two key tiles of a query tile
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    if (k0 + i > qpos) sv[i] = 0xff800000u;   // -inf
                    mh = fmaxf(mh, __uint_as_float(sv[i]));
                }
            } else {
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[i]));
                mh = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            xm[r][half] = mh;
            pair_sync();
            const float mx = fmaxf(xm[r][0], xm[r][1]);       // the same value in both threads of the row
            pair_sync();                                      // both have read it: the slot is free for the next tile
            // tcgen05.ld / st are warp-wide: the warp rescales together, rows that need none by 1
            const bool grow = (mx - m) * c > 8.0f;            // also true for the first tile (m = -inf)
            // o_full completes once per key tile and is waited on by parity, so every thread consumes EVERY
            // phase, in order (a parity wait that is two phases behind returns at once): phase j - 1 here if
            // the accumulator is rescaled, else just before this tile's probabilities are handed over.
            bool seen_prev = j == 0;
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? fast_exp2((m - mx) * c) : 1.0f;   // 0 for the first tile
                if (j > 0) {
                    // the previous P V product must have landed before the accumulator is touched
                    ok = ok && mbar_wait(o_full, (uint32_t)(j - 1) & 1u, status);
                    seen_prev = true;
                    tc_fence_after();
#pragma unroll
                    for (int cb = 0; cb < 2; ++cb) {
                        uint32_t v[32];
                        tmem_ld32(tmem_o + lane_off + col_off + cb * 32, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st32(tmem_o + lane_off + col_off + cb * 32, v);
                    }
                    tc_fence_before();
                }
                l *= alpha;
                if (grow) m = mx;
            }
            const float mc = m * c;
            // (S[st] last held the probabilities of tile j - 2; their product was issued before the Q K^T of this tile)
            // probabilities -> bf16 pairs -> A operand of the P V product in tensor memory; this thread's 64 keys
            // are 32 packed columns
            float rs = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), c, -mc));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), c, -mc));
                rs += p0 + p1;
                pk[i] = pack_bf16x2(p0, p1);
            }
            // into the columns the scores of keys 0-63 came from (both threads of the row have read theirs: the
            // exchange above lies in between); 64 keys of the row are 32 columns
            tmem_st32(tmem_base + st * 128 + lane_off + half * 32, pk);
            l += rs;
            if (!seen_prev) ok = ok && mbar_wait(o_full, (uint32_t)(j - 1) & 1u, status);   // P V of tile j - 1 (precedes this tile's anyway)
            tc_fence_before();
            mbar_arrive(&p_full[st]);
        }
        // the last P V product, then out = O / l (l = the sum of the two half-row sums)
        ok = ok && mbar_wait(o_full, (uint32_t)(nt - 1) & 1u, status);
        tc_fence_after();
        xm[r][half] = l;
        pair_sync();
        const float inv = 1.0f / (xm[r][0] + xm[r][1]);
        bf16* orow = out + (size_t)(q0 + r) * QSZ + head * D + half * 64;
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_off + col_off + cb * 32, v);
            if (q0 + r < S) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    reinterpret_cast<uint4*>(orow + cb * 32)[q] =
                        make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]) * inv, __uint_as_float(v[8 * q + 1]) * inv),
                                   pack_bf16x2(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv),
                                   pack_bf16x2(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv),
                                   pack_bf16x2(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv));
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TA_TMEM_COLS);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MapKey {
    const void* ptr; uint64_t rows, cols, ld; uint32_t box_rows;
    uint64_t planes, plane_ld;           // 0, 0 for a matrix
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && planes == o.planes && plane_ld == o.plane_ld;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h ^= k.rows * 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= k.cols * 0xc2b2ae3d27d4eb4full + (h << 6) + (h >> 2);
        h ^= (k.ld * 31 + k.box_rows) + (h << 6) + (h >> 2);
        h ^= (k.planes * 0x9e3779b97f4a7c15ull + k.plane_ld) + (h << 6) + (h >> 2);
        return h;
    }
};
static std::mutex g_map_mu;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static EncodeTiledFn g_encode = nullptr;

// Tensor map of a row-major bf16 matrix [rows, cols] with leading dimension ld
// (elements); box = 64 columns x box_rows rows, 128-byte swizzle, zero fill
// outside the matrix.  Maps are cached: weight matrices never move.
// planes > 0: a stack of `planes` such matrices, plane_ld elements apart (a third coordinate selects the plane,
// and rows beyond `rows` of a plane are filled with zeros instead of running into the next plane).
static int get_map(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, CUtensorMap* out, uint64_t planes = 0,
                   uint64_t plane_ld = 0) {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return (int)e;
        if (!fn || qres != cudaDriverEntryPointSuccess) return MQ_ERR_UNSUPPORTED;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const MapKey key{ptr, rows, cols, ld, box_rows, planes, plane_ld};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return MQ_OK; }
    if (g_maps.size() > 4096) g_maps.clear();
    const cuuint64_t dims[3] = {cols, rows, planes};
    const cuuint64_t strides[2] = {ld * 2, plane_ld * 2};
    const cuuint32_t box[3] = {GM_BK, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    const CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, planes > 0 ? 3 : 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MQ_ERR_BAD_ARG;
    g_maps.emplace(key, m);
    *out = m;
    return MQ_OK;
}

template <int BN, int EPI, int MT = 1>
static int launch_gemm(const bf16* A, int lda, const bf16* B, const bf16* B2, bf16* C, const bf16* R, int M, int N, int K, int ldc,
                       unsigned int* status, cudaStream_t stream, const bf16* B3 = nullptr, int rows0 = 0, int rows1 = 0, int ksplit = 1,
                       int drop_kb = -1, bool early_b = true) {
    // early_b: B (B2, B3) are weights, never written by work on this stream; false for caller-supplied operands
    // rows0 > 0: B, B2, B3 hold rows0, rows1 and N - rows0 - rows1 output columns (concatenated along N)
    using Cfg = GemmCfg<BN, EPI, MT>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm<BN, EPI, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    if (N % BN != 0 || K % GM_BK != 0) return MQ_ERR_BAD_ARG;
    CUtensorMap ma, mb, mb2;
    int rc = get_map(A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GM_BM, &ma);
    if (rc != MQ_OK) return rc;
    const bool concat = rows0 > 0;
    if (concat && (rows0 % BN || rows1 % BN || EPI == EPI_SWIGLU)) return MQ_ERR_BAD_ARG;
    rc = get_map(B, (uint64_t)(concat ? rows0 : N), (uint64_t)K, (uint64_t)K, BN, &mb);
    if (rc != MQ_OK) return rc;
    mb2 = mb;
    CUtensorMap mb3 = mb;
    if (EPI == EPI_SWIGLU) {
        rc = get_map(B2, (uint64_t)N, (uint64_t)K, (uint64_t)K, BN, &mb2);
        if (rc != MQ_OK) return rc;
    } else if (concat) {
        rc = get_map(B2, (uint64_t)rows1, (uint64_t)K, (uint64_t)K, BN, &mb2);
        if (rc != MQ_OK) return rc;
        rc = get_map(B3, (uint64_t)(N - rows0 - rows1), (uint64_t)K, (uint64_t)K, BN, &mb3);
        if (rc != MQ_OK) return rc;
    }
    if (ksplit < 1 || (ksplit > 1 && EPI != EPI_PARTIAL) || K / GM_BK < ksplit) return MQ_ERR_BAD_ARG;
    dim3 grid(N / BN, (M + GM_BM * MT - 1) / (GM_BM * MT), ksplit);
    launch_pdl(k_gemm<BN, EPI, MT>, dim3(grid), dim3(GM_TILE_THREADS), Cfg::SMEM, stream, ma, mb, mb2, mb3, concat ? rows0 / BN : (1 << 30), concat ? rows1 / BN : 0,
                                                             C, R, M, N, K, ldc, status, drop_kb, early_b ? 1 : 0);
    return (int)cudaGetLastError();
}

// Skinny path: part[ks][M][ldp] = X[M,K] * [W0;W1;W2][.,K]^T, K split in `ksplit` slices.
template <int MPAD>
static int launch_skinny_t(const bf16* const* W, const int* rowsW, int nW, const bf16* X, int ldx, float* part, int M, int K, int ksplit,
                           unsigned int* status, cudaStream_t stream) {
    constexpr int X_STRIDE = ((MPAD * GM_BK * 2) + 1023) & ~1023;
    const size_t smem = (size_t)SK_MAXKB * (128 * GM_BK * 2 + X_STRIDE) + 1024 + 256;
    static bool attr_set[64] = {false};
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm_skinny<MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    const int kb = K / GM_BK;
    if (K % GM_BK != 0 || kb % ksplit != 0 || kb / ksplit > SK_MAXKB) return MQ_ERR_BAD_ARG;
    CUtensorMap mw[3], mx;
    int tiles[3] = {0, 0, 0}, ldp = 0;
    for (int i = 0; i < 3; ++i) {
        const int j = i < nW ? i : 0;
        if (rowsW[j] % 128 != 0) return MQ_ERR_BAD_ARG;
        int rc = get_map(W[j], (uint64_t)rowsW[j], (uint64_t)K, (uint64_t)K, 128, &mw[i]);
        if (rc != MQ_OK) return rc;
        if (i < nW) { tiles[i] = rowsW[i] / 128; ldp += rowsW[i]; }
    }
    int rc = get_map(X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, MPAD, &mx);
    if (rc != MQ_OK) return rc;
    dim3 grid(tiles[0] + tiles[1] + tiles[2], ksplit);
    // A grid of at most one CTA per SM asks for the full ring, so that no two of its CTAs share an SM; a larger
    // one (gate|up: 48 tiles x 4 K slices = 192 CTAs) asks for what its k-blocks need and runs in one round.
    const size_t smem_exact = (size_t)(kb / ksplit) * (128 * GM_BK * 2 + X_STRIDE) + 1024 + 256;
    const size_t smem_used = (int)(grid.x * grid.y) > sms[dev] ? smem_exact : smem;
    launch_pdl(k_gemm_skinny<MPAD>, dim3(grid), dim3(GM_THREADS), smem_used, stream, mw[0], mw[1], mw[2], tiles[0], tiles[1], mx, part, M, ldp, kb / ksplit, status);
    return (int)cudaGetLastError();
}
static int launch_skinny(const bf16* const* W, const int* rowsW, int nW, const bf16* X, int ldx, float* part, int M, int K, int ksplit,
                         unsigned int* status, cudaStream_t stream) {
    if (M <= 16) return launch_skinny_t<16>(W, rowsW, nW, X, ldx, part, M, K, ksplit, status, stream);
    if (M <= 32) return launch_skinny_t<32>(W, rowsW, nW, X, ldx, part, M, K, ksplit, status, stream);
    if (M <= 64) return launch_skinny_t<64>(W, rowsW, nW, X, ldx, part, M, K, ksplit, status, stream);
    return MQ_ERR_BAD_ARG;
}

// defined in decode.cu: final RMSNorm + LM head + arg-max on buf->hidden
int launch_lmhead_only(const MqModel* model, const MqDecodeBuffers* buf, int* out_token, float* logits, cudaStream_t stream);

__global__ void k_pf_copy_row(const bf16* __restrict__ src, bf16* __restrict__ dst) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    reinterpret_cast<uint4*>(dst)[threadIdx.x] = reinterpret_cast<const uint4*>(src)[threadIdx.x];
}

// dst[b] = src[last packed row of sequence b]
__global__ void k_pf_gather_last(const bf16* __restrict__ src, const int* __restrict__ seq_row0, const int* __restrict__ seq_len,
                                 bf16* __restrict__ dst) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    const int b = blockIdx.x;
    const size_t row = (size_t)seq_row0[b] + (size_t)seq_len[b] - 1;
    reinterpret_cast<uint4*>(dst + (size_t)b * H)[threadIdx.x] = reinterpret_cast<const uint4*>(src + row * H)[threadIdx.x];
}

}  // namespace mq

namespace mq {

// ---------------------------------------------------------------- batched decode (one new token per sequence)
// One CTA per (sequence, kv head); the two query heads share the K/V stream.  Each warp owns
// the 16-position tiles warp, warp + 12, .. of the sequence and streams them through its own
// two-stage ring of padded rows in shared memory (16-byte cp.async, the next tile in flight
// while this one is multiplied, no block barrier inside the loop; twelve warps per SM rather
// than eight with deeper rings, because the per-tile chain of dependent instructions, not
// the bytes in flight, bounds a warp; one 256-byte bulk copy per row instead of sixteen
// cp.async was measured slower: 3.07 vs 2.81 ms per step at batch 64).  Per tile: scores = K_tile . q on mma.sync (positions
// are M, the two heads two of the eight N columns), softmax of the tile, P rounded to bf16,
// out += P . V_tile (ldmatrix.trans on V).  About a sixth of the instructions of an fp32-FMA
// loop over the same bytes, which is what bounded the FMA version at 2.7 TB/s.
constexpr int BD_STAGES = 2, BD_LD = D + 8;                                     // per warp: 2 stages x 8.5 KB
constexpr int BD_STAGE_ELEMS = 2 * 16 * BD_LD;                                  // K tile then V tile
// Two shapes: twelve warps, one CTA per SM (209 KB), or six warps, two CTAs per SM (105 KB each).  The
// SM streams with twelve warps either way; bd_shape() below says which is used when.
constexpr size_t bd_smem_bytes(int warps) { return (size_t)warps * BD_STAGES * BD_STAGE_ELEMS * 2 + 2 * D * 2 + warps * 32 * 2; }
constexpr int BD_MAX_PARTS = 4;                                                 // CTAs that may share one item's keys
constexpr int BD_PART = D + 2;                                                  // m, l, acc[128] of one head of one part
// FP8 cache: a warp's ring holds the raw e4m3 rows (K 16 x 128 bytes, then V), two stages, followed
// by ONE padded f16 tile pair the current stage is expanded into before it is multiplied
constexpr int BD8_RAW = 2 * 16 * D;                                             // bytes per raw stage
constexpr int BD8_WARP_BYTES = BD_STAGES * BD8_RAW + BD_STAGE_ELEMS * 2;
static_assert(BD8_WARP_BYTES <= BD_STAGES * BD_STAGE_ELEMS * 2, "the fp8 ring fits the bf16 ring");

__device__ __forceinline__ void bd_load_tile(bf16* stage, const bf16* kb, const bf16* vb, int tile, int len, int lane) {
    // 16 rows x 16 chunks of 16 bytes for K and the same for V: 16 copies per lane.  Rows past
    // the end of the sequence re-read the last row (their probabilities are zero).
    // copy i of a lane is chunk (lane & 15) of row 2 * i + (lane >> 4)
    const int c8 = (lane & 15) * 8, r0 = lane >> 4;
    bf16* sdst = stage + r0 * BD_LD + c8;
    const int last = len - 1 - tile * 16 - r0;            // copies with 2 * i > last re-read the last row
    const size_t gbase = (size_t)(tile * 16 + r0) * D + c8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const size_t goff = gbase + (size_t)min(2 * i, last) * D;
        cp_async16(sdst + 2 * i * BD_LD, kb + goff);
        cp_async16(sdst + (16 + 2 * i) * BD_LD, vb + goff);
    }
}
// e4m3 rows: 16 rows x 8 chunks of 16 bytes for K and for V, 8 copies per lane; copy i of a lane
// is chunk (lane & 7) of row 4 * (i & 3) + (lane >> 3) of K (i < 4) or V
__device__ __forceinline__ void bd_load_tile_fp8(uint8_t* raw, const uint8_t* kb, const uint8_t* vb, int tile, int len, int lane) {
    const int c16 = (lane & 7) * 16, r0 = lane >> 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = 4 * i + r0;
        const size_t goff = (size_t)min(tile * 16 + r, len - 1) * D + c16;
        cp_async16(raw + r * D + c16, kb + goff);
        cp_async16(raw + 16 * D + r * D + c16, vb + goff);
    }
}
// the raw stage -> padded f16 tiles (same chunk assignment as the copies)
__device__ __forceinline__ void bd_expand_tile_fp8(const uint8_t* raw, bf16* tile16, int lane) {
    const int c16 = (lane & 7) * 16, r0 = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = 4 * (i & 3) + r0 + (i >> 2) * 16;      // rows 16..31 are V
        const uint4 w = *reinterpret_cast<const uint4*>(raw + r * D + c16);
        uint4 a, b;
        fp8x16_to_f16x16(w, a, b);
        uint4* dst = reinterpret_cast<uint4*>(tile16 + r * BD_LD + c16);
        dst[0] = a;
        dst[1] = b;
    }
}

// FP8 = true: K and V are read from the e4m3 shadow cache (k8 / v8, one scale per sequence, layer
// and kv head: scores are multiplied by the K scale, the output by the V scale; reference:
// decode attention with KV_FP8, csrc/megakernel/split_decode_gemm.cu:950-1310).  The row of
// the new position was written to the bf16 cache by the preceding kernel; this CTA quantises
// it into the shadow cache first (split_decode_gemm.cu:487-493).
// qk.part != nullptr: the step's q|k|v rows are still the fp32 planes of the K-split projection; the CTA sums
// its item's four heads itself (two query heads, and in the part that holds the new position the K and V
// head), applies QK-norm + RoPE with the arithmetic of k_pf_qknorm_rope and writes the new K / V row into
// the cache, so that kernel is not launched.
// One-dimensional grid: CTAs 0 .. n_full - 1 take one (sequence, kv head) item each; the remaining items
// are split over p_tail CTAs each (CTA n_full + r: item n_full + r / p_tail, part r % p_tail).  The CTAs
// of a split item write their (m, l, acc) to `parts` and take a ticket, and the one that takes the last
// merges them (no CTA waits for another).  tickets: one zero-initialised counter per item, reset by the merger.
struct BdQkFuse {
    const float* part;        // [ksplit][M][QKV] fp32 planes of the q|k|v projection, or nullptr
    int ksplit, M;
    const bf16* wq; const bf16* wk; const bf16* cos; const bf16* sin;
};
template <bool FP8, int WARPS>
__device__ __forceinline__ void bd_attention_body(const bf16* __restrict__ qkv, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                                  bf16* __restrict__ out, const int* __restrict__ positions, int layer, int max_seq,
                                                  size_t seq_stride, uint8_t* __restrict__ k8, uint8_t* __restrict__ v8,
                                                  const float* __restrict__ k_scale, const float* __restrict__ v_scale, int scale_stride,
                                                  float* __restrict__ parts, unsigned int* __restrict__ tickets, int n_full, int p_tail,
                                                  const BdQkFuse& qk) {
    constexpr int BD_THREADS = WARPS * 32;
    const int cta = (int)blockIdx.x;
    const int item_i = cta < n_full ? cta : n_full + (cta - n_full) / p_tail;
    const int part = cta < n_full ? 0 : (cta - n_full) % p_tail;
    const int nparts = cta < n_full ? 1 : p_tail;
    const int b = item_i / NKV, g = item_i % NKV;
    // the scales are set by the quantise kernel before the first step and constant afterwards
    float ks = 1.f, vs = 1.f;
    if constexpr (FP8) {
        ks = kv_fp8_scale_guard(k_scale[(size_t)b * scale_stride + layer * NKV + g]);
        vs = kv_fp8_scale_guard(v_scale[(size_t)b * scale_stride + layer * NKV + g]);
    }
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    extern __shared__ __align__(128) uint8_t bd_smem[];
    bf16* ring = reinterpret_cast<bf16*>(bd_smem);                                    // [12 warps][2 stages][K 16 rows | V 16 rows][BD_LD]
    bf16* qs = ring + (size_t)(BD_THREADS / 32) * BD_STAGES * BD_STAGE_ELEMS;         // [2][D]
    bf16* ps = qs + 2 * D;                                                            // [12 warps][2][16]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = min(max(positions[b], 0), max_seq - 1);
    const int len = pos + 1;
    const int ntiles_all = (len + 15) >> 4;
    // this CTA's share of the item's key tiles: [tile_lo, ntiles)
    const int tile_lo = (int)(((long long)part * ntiles_all) / nparts);
    const int ntiles = (int)(((long long)(part + 1) * ntiles_all) / nparts);
    const bool has_new = part == nparts - 1;                 // the part that holds the new position's tile
    const size_t head_off = (size_t)b * seq_stride + ((size_t)(layer * NKV + g) * max_seq) * D;
    const bf16* kb = k_cache + head_off;
    const bf16* vb = v_cache + head_off;
    bf16* wring = ring + (size_t)warp * BD_STAGES * BD_STAGE_ELEMS;
    uint8_t* wraw = bd_smem + (size_t)warp * BD8_WARP_BYTES;                          // FP8: [2][raw stage] | f16 tile pair
    bf16* wtile = reinterpret_cast<bf16*>(wraw + BD_STAGES * BD8_RAW);
    const uint8_t* k8b = FP8 ? k8 + head_off : nullptr;
    const uint8_t* v8b = FP8 ? v8 + head_off : nullptr;

    // The first tile of this warp is requested before anything else.  The tile that holds the new position
    // waits for the block barrier below where this CTA writes that row itself (FP8: the quantised row written
    // by threads 0..63; fused QK-norm: the bf16 row written by warps 2 and 3).
    const bool fused = qk.part != nullptr;
    const bool defer_new = has_new && (FP8 || fused);
#pragma unroll
    for (int s = 0; s < BD_STAGES - 1; ++s) {
        const int t = tile_lo + warp + s * (BD_THREADS / 32);
        if (t < ntiles && !(defer_new && t == ntiles - 1)) {
            if constexpr (FP8) bd_load_tile_fp8(wraw + s * BD8_RAW, k8b, v8b, t, len, lane);
            else bd_load_tile(wring + s * BD_STAGE_ELEMS, kb, vb, t, len, lane);
        }
        cp_async_commit();
    }
    if (fused) {
        // warp 0, 1: query heads 2 g, 2 g + 1 -> qs; warp 2: the new K row; warp 3: the new V row (both into the cache)
        if (warp < 2 || (warp < 4 && has_new)) {
            const size_t plane = (size_t)qk.M * QKV;
            const int col0 = warp < 2 ? (2 * g + warp) * D : warp == 2 ? QSZ + g * D : QSZ + KVSZ + g * D;
            const size_t i0 = (size_t)b * QKV + col0;
            if (warp == 3) {
                float f[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) f[e] = sum_splits(qk.part, qk.ksplit, plane, i0 + 4 * lane + e);
                *reinterpret_cast<uint2*>(const_cast<bf16*>(vb) + (size_t)pos * D + 4 * lane) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
            } else {
                // the norm weights and the position's cos / sin rows are requested together with the planes
                const bf16* wn = warp < 2 ? qk.wq : qk.wk;
                const bf16* cosr = qk.cos + (size_t)pos * D;
                const bf16* sinr = qk.sin + (size_t)pos * D;
                const uint32_t wl = *reinterpret_cast<const uint32_t*>(wn + 2 * lane), wh = *reinterpret_cast<const uint32_t*>(wn + 64 + 2 * lane);
                const uint32_t cl = *reinterpret_cast<const uint32_t*>(cosr + 2 * lane), chh = *reinterpret_cast<const uint32_t*>(cosr + 64 + 2 * lane);
                const uint32_t sl = *reinterpret_cast<const uint32_t*>(sinr + 2 * lane), sh = *reinterpret_cast<const uint32_t*>(sinr + 64 + 2 * lane);
                float xl[2], xh[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    xl[e] = rbf(sum_splits(qk.part, qk.ksplit, plane, i0 + 2 * lane + e));
                    xh[e] = rbf(sum_splits(qk.part, qk.ksplit, plane, i0 + 64 + 2 * lane + e));
                }
                float ss = xl[0] * xl[0] + xl[1] * xl[1] + xh[0] * xh[0] + xh[1] * xh[1];
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
                const float wlo[2] = {bf_lo(wl), bf_hi(wl)}, whi[2] = {bf_lo(wh), bf_hi(wh)};
                const float clo[2] = {bf_lo(cl), bf_hi(cl)}, chi[2] = {bf_lo(chh), bf_hi(chh)};
                const float slo[2] = {bf_lo(sl), bf_hi(sl)}, shi[2] = {bf_lo(sh), bf_hi(sh)};
                float lo[2], hi[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float nl = rbf(wlo[e] * rbf(xl[e] * r));
                    const float nh = rbf(whi[e] * rbf(xh[e] * r));
                    lo[e] = rbf(rbf(nl * clo[e]) + rbf(-nh * slo[e]));
                    hi[e] = rbf(rbf(nh * chi[e]) + rbf(nl * shi[e]));
                }
                if (warp < 2) {
                    bf16* qd = qs + warp * D;
                    *reinterpret_cast<uint32_t*>(qd + 2 * lane) = FP8 ? pack_f16x2(lo[0], lo[1]) : pack_bf16x2(lo[0], lo[1]);
                    *reinterpret_cast<uint32_t*>(qd + 64 + 2 * lane) = FP8 ? pack_f16x2(hi[0], hi[1]) : pack_bf16x2(hi[0], hi[1]);
                } else {
                    bf16* kd = const_cast<bf16*>(kb) + (size_t)pos * D;
                    *reinterpret_cast<uint32_t*>(kd + 2 * lane) = pack_bf16x2(lo[0], lo[1]);
                    *reinterpret_cast<uint32_t*>(kd + 64 + 2 * lane) = pack_bf16x2(hi[0], hi[1]);
                }
            }
        }
        if constexpr (FP8) __syncthreads();   // the bf16 row is complete before threads 0..63 quantise it
    }
    if constexpr (FP8) {
        if (tid < 64 && has_new) {
            const int e4 = 4 * (tid & 31);
            const bool isk = tid < 32;
            const uint2 u = *reinterpret_cast<const uint2*>((isk ? kb : vb) + (size_t)pos * D + e4);
            const float inv = 1.0f / (isk ? ks : vs);
            *reinterpret_cast<uint32_t*>((isk ? k8 : v8) + head_off + (size_t)pos * D + e4) =
                f32x4_to_fp8x4(bf_lo(u.x) * inv, bf_hi(u.x) * inv, bf_lo(u.y) * inv, bf_hi(u.y) * inv);
            __threadfence_block();
        }
    }
    if (!fused && tid >= 64 && tid < 96) {
        const int t8 = tid - 64;
        uint4 q = *reinterpret_cast<const uint4*>(qkv + (size_t)b * QKV + 2 * g * D + t8 * 8);
        if constexpr (FP8) {   // f16 tiles are multiplied with an f16 query
            q.x = pack_f16x2(bf_lo(q.x), bf_hi(q.x)); q.y = pack_f16x2(bf_lo(q.y), bf_hi(q.y));
            q.z = pack_f16x2(bf_lo(q.z), bf_hi(q.z)); q.w = pack_f16x2(bf_lo(q.w), bf_hi(q.w));
        }
        *reinterpret_cast<uint4*>(qs + t8 * 8) = q;
    }
    __syncthreads();
    if (FP8 || fused) {
        const int tl = ntiles - 1 - tile_lo;                  // the deferred tile, counted from this part's first
        if (defer_new && tl >= 0 && tl < (BD_STAGES - 1) * (BD_THREADS / 32) && warp == tl % (BD_THREADS / 32)) {
            if constexpr (FP8) bd_load_tile_fp8(wraw + (tl / (BD_THREADS / 32)) * BD8_RAW, k8b, v8b, ntiles - 1, len, lane);
            else bd_load_tile(wring + (tl / (BD_THREADS / 32)) * BD_STAGE_ELEMS, kb, vb, ntiles - 1, len, lane);
        }
        cp_async_commit();
    }

    const int gi = lane >> 2, ti = lane & 3;
    const float scale = 0.08838834764831845f * ks;  // 1/sqrt(128) (x the K scale)
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    uint32_t qb[D / 16][2];   // B fragments of the two query heads (columns 2..7 are zero)
    {
        const uint32_t qaddr = smem_u32(qs) + (uint32_t)((gi & 1) * D + 2 * ti) * 2u;
#pragma unroll
        for (int ks16 = 0; ks16 < D / 16; ++ks16) {
            qb[ks16][0] = gi < 2 ? lds32(qaddr + ks16 * 32) : 0u;
            qb[ks16][1] = gi < 2 ? lds32(qaddr + ks16 * 32 + 16) : 0u;
        }
    }
    bf16* pw = ps + warp * 32;
    int it = 0;
    for (int tile = tile_lo + warp; tile < ntiles; tile += BD_THREADS / 32, ++it) {
        cp_async_wait<BD_STAGES - 2>();   // this tile has landed (one younger group may be in flight)
        __syncwarp();
        const bf16* st = FP8 ? wtile : wring + (it % BD_STAGES) * BD_STAGE_ELEMS;
        // the stage consumed in the previous iteration is free: request the next tile of this warp
        {
            const int tn = tile + (BD_STAGES - 1) * (BD_THREADS / 32);
            if (tn < ntiles) {
                if constexpr (FP8) bd_load_tile_fp8(wraw + ((it + BD_STAGES - 1) % BD_STAGES) * BD8_RAW, k8b, v8b, tn, len, lane);
                else bd_load_tile(wring + ((it + BD_STAGES - 1) % BD_STAGES) * BD_STAGE_ELEMS, kb, vb, tn, len, lane);
            }
            cp_async_commit();
        }
        if constexpr (FP8) {
            bd_expand_tile_fp8(wraw + (it % BD_STAGES) * BD8_RAW, wtile, lane);
            __syncwarp();
        }
        const uint32_t rowoff = (uint32_t)(((lane & 15) * BD_LD + (lane >> 4) * 8) * 2);
        const uint32_t kaddr = smem_u32(st) + rowoff, vaddr = kaddr + 16 * BD_LD * 2;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks16 = 0; ks16 < D / 16; ++ks16) {
            uint32_t af[4];
            ldsm4(af, kaddr + ks16 * 32);
            mma16816_sel<FP8>(c, af, qb[ks16][0], qb[ks16][1]);
        }
        // lanes with ti == 0 hold head 0 / head 1 of positions gi (c[0], c[1]) and gi + 8 (c[2], c[3])
        const int p_lo = tile * 16 + gi, p_hi = p_lo + 8;
        const bool own = ti == 0;
        const float s00 = (own && p_lo < len) ? c[0] * scale : -1e30f, s01 = (own && p_lo < len) ? c[1] * scale : -1e30f;
        const float s10 = (own && p_hi < len) ? c[2] * scale : -1e30f, s11 = (own && p_hi < len) ? c[3] * scale : -1e30f;
        float t0 = fmaxf(s00, s10), t1 = fmaxf(s01, s11);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, off));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, off));
        }
        t0 = __shfl_sync(0xffffffffu, t0, 0);
        t1 = __shfl_sync(0xffffffffu, t1, 0);
        const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
        const float cr0 = expf(m0 - mn0), cr1 = expf(m1 - mn1);
        m0 = mn0; m1 = mn1;
        const float e00 = (own && p_lo < len) ? expf(s00 - m0) : 0.f, e01 = (own && p_lo < len) ? expf(s01 - m1) : 0.f;
        const float e10 = (own && p_hi < len) ? expf(s10 - m0) : 0.f, e11 = (own && p_hi < len) ? expf(s11 - m1) : 0.f;
        float u0 = e00 + e10, u1 = e01 + e11;
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            u0 += __shfl_xor_sync(0xffffffffu, u0, off);
            u1 += __shfl_xor_sync(0xffffffffu, u1, off);
        }
        l0 = l0 * cr0 + __shfl_sync(0xffffffffu, u0, 0);
        l1 = l1 * cr1 + __shfl_sync(0xffffffffu, u1, 0);
        if (own) {
            if constexpr (FP8) {   // probabilities rounded to bf16 as on the bf16 path (exact in f16: 8 significant bits, e <= 1)
                __half* ph = reinterpret_cast<__half*>(pw);
                ph[gi] = __float2half_rn(rbf(e00)); ph[gi + 8] = __float2half_rn(rbf(e10));
                ph[16 + gi] = __float2half_rn(rbf(e01)); ph[16 + gi + 8] = __float2half_rn(rbf(e11));
            } else {
                pw[gi] = __float2bfloat16_rn(e00); pw[gi + 8] = __float2bfloat16_rn(e10);
                pw[16 + gi] = __float2bfloat16_rn(e01); pw[16 + gi + 8] = __float2bfloat16_rn(e11);
            }
        }
        __syncwarp();
        uint32_t pa[4] = {0u, 0u, 0u, 0u};   // A = P: row gi is head gi (rows 2..15 are zero)
        if (gi < 2) {
            pa[0] = *reinterpret_cast<const uint32_t*>(pw + gi * 16 + 2 * ti);
            pa[2] = *reinterpret_cast<const uint32_t*>(pw + gi * 16 + 8 + 2 * ti);
        }
        if (cr0 != 1.f || cr1 != 1.f) {   // the same for every lane
            const float crg = gi == 0 ? cr0 : cr1;
#pragma unroll
            for (int j = 0; j < 16; ++j) { o[j][0] *= crg; o[j][1] *= crg; }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t bv[4];
            ldsm4_t(bv, vaddr + j * 32);
            mma16816_sel<FP8>(o[2 * j], pa, bv[0], bv[1]);
            mma16816_sel<FP8>(o[2 * j + 1], pa, bv[2], bv[3]);
        }
        __syncwarp();
    }
    cp_async_wait_all();
    __syncthreads();   // every warp is done with its ring: the merge buffers reuse it
    float* s_acc = reinterpret_cast<float*>(bd_smem);          // [WARPS][2][D]
    float* s_m = s_acc + WARPS * 2 * D;                        // [WARPS][2]
    float* s_l = s_m + WARPS * 2;                              // [WARPS][2]
    if (lane == 0) { s_m[warp * 2] = m0; s_m[warp * 2 + 1] = m1; s_l[warp * 2] = l0; s_l[warp * 2 + 1] = l1; }
    if (gi < 2) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            *reinterpret_cast<float2*>(s_acc + (warp * 2 + gi) * D + j * 8 + 2 * ti) = make_float2(o[j][0], o[j][1]);
    }
    __syncthreads();
    const size_t item = (size_t)b * NKV + g;
    for (int idx = tid; idx < 2 * D; idx += BD_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        float M = -1e30f;
#pragma unroll
        for (int w8 = 0; w8 < WARPS; ++w8) M = fmaxf(M, s_m[w8 * 2 + hh]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < WARPS; ++w8) {
            const float f = expf(s_m[w8 * 2 + hh] - M);
            den = fmaf(s_l[w8 * 2 + hh], f, den);
            num = fmaf(s_acc[(w8 * 2 + hh) * D + d], f, num);
        }
        if (nparts == 1) {
            out[(size_t)b * QSZ + (2 * g + hh) * D + d] = __float2bfloat16_rn(num / den * vs);
        } else {
            float* pp = parts + ((item * BD_MAX_PARTS + part) * 2 + hh) * BD_PART;
            pp[2 + d] = num;
            if (d == 0) { pp[0] = M; pp[1] = den; }
        }
    }
    if (nparts == 1) return;
    // the block barrier orders every thread's partial before thread 0's release; the CTA that takes the
    // last ticket acquires the others' partials with the same instruction
    __shared__ int s_last;
    __syncthreads();
    if (tid == 0) {
        unsigned int t;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(t) : "l"(tickets + item) : "memory");
        s_last = (t == (unsigned int)(nparts - 1));
        if (s_last) tickets[item] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    for (int idx = tid; idx < 2 * D; idx += BD_THREADS) {
        const int hh = idx >> 7, d = idx & 127;
        const float* pb = parts + (item * BD_MAX_PARTS * 2 + hh) * BD_PART;
        float mj[BD_MAX_PARTS], M = -1e30f;
#pragma unroll
        for (int j = 0; j < BD_MAX_PARTS; ++j) {
            mj[j] = j < nparts ? ld_cg_f32(pb + (size_t)j * 2 * BD_PART) : -1e30f;
            M = fmaxf(M, mj[j]);
        }
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int j = 0; j < BD_MAX_PARTS; ++j) {
            if (j < nparts) {
                const float f = expf(mj[j] - M);
                den = fmaf(ld_cg_f32(pb + (size_t)j * 2 * BD_PART + 1), f, den);
                num = fmaf(ld_cg_f32(pb + (size_t)j * 2 * BD_PART + 2 + d), f, num);
            }
        }
        out[(size_t)b * QSZ + (2 * g + hh) * D + d] = __float2bfloat16_rn(num / den * vs);
    }
}

template <bool FP8, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 6 ? 2 : 1)
k_bd_attention(const bf16* __restrict__ qkv, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, bf16* __restrict__ out,
               const int* __restrict__ positions, int layer, int max_seq, size_t seq_stride, uint8_t* __restrict__ k8, uint8_t* __restrict__ v8,
               const float* __restrict__ k_scale, const float* __restrict__ v_scale, int scale_stride, float* __restrict__ parts,
               unsigned int* __restrict__ tickets, int n_full, int p_tail, const BdQkFuse qk) {
    bd_attention_body<FP8, WARPS>(qkv, k_cache, v_cache, out, positions, layer, max_seq, seq_stride, k8, v8, k_scale, v_scale, scale_stride, parts,
                                  tickets, n_full, p_tail, qk);
}

// out_tokens[b] = lowest index of the maximum bf16 logit of row b; positions[b] += 1.
__global__ void __launch_bounds__(1024) k_bd_argmax_advance(const bf16* __restrict__ logits, int vocab, int* __restrict__ out_tokens,
                                                            int* __restrict__ positions, float* __restrict__ logits_f32) {
    pdl_trigger();   // the next grid may be scheduled already (it waits the same way)
    pdl_wait();      // launched with programmatic stream serialisation: the preceding grid has completed
    __shared__ unsigned long long s_best[32];
    const int b = blockIdx.x, tid = threadIdx.x;
    const bf16* row = logits + (size_t)b * vocab;
    unsigned long long best = 0ull;
    // 16-byte loads, eight logits each (the vocabulary is a multiple of 128 and rows are 16-byte aligned)
    const uint4* row4 = reinterpret_cast<const uint4*>(row);
    for (int i4 = tid; i4 < vocab / 8; i4 += blockDim.x) {
        const uint4 q = row4[i4];
        const uint32_t wds[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v = (e & 1) ? bf_hi(wds[e >> 1]) : bf_lo(wds[e >> 1]);
            const int i = i4 * 8 + e;
            if (logits_f32) logits_f32[(size_t)b * vocab + i] = v;
            uint32_t u = __float_as_uint(v);
            u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            const unsigned long long key = ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
            best = key > best ? key : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((tid & 31) == 0) s_best[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = s_best[i] > best ? s_best[i] : best;
        out_tokens[b] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        positions[b] += 1;
    }
}

}  // namespace mq

using namespace mq;

// kernels of one prefill (at most: the split-K path needs one norm kernel fewer per layer after the first)
extern "C" int mq_prefill_launch_count(int num_layers) { return 1 + num_layers * 8 + 2; }

// C[M,N] = A[M,K] * B[N,K]^T on the tcgen05 path (bf16 in/out, fp32 accumulate);
// optional residual R (same shape and leading dimension as C, may alias C).
extern "C" int mq_launch_gemm_bf16(const void* A, int lda, const void* B, void* C, const void* R, int M, int N, int K, int ldc,
                                   unsigned int* status, void* stream) {
    if (!A || !B || !C || !status || M <= 0 || N <= 0 || K <= 0) return MQ_ERR_BAD_ARG;
    if (lda % 8 != 0 || ldc % 8 != 0) return MQ_ERR_ALIGNMENT;
    if (R) return launch_gemm<128, EPI_RESID>((const bf16*)A, lda, (const bf16*)B, nullptr, (bf16*)C, (const bf16*)R, M, N, K, ldc, status, (cudaStream_t)stream,
                                              nullptr, 0, 0, 1, -1, false);
    return launch_gemm<128, EPI_STORE>((const bf16*)A, lda, (const bf16*)B, nullptr, (bf16*)C, nullptr, M, N, K, ldc, status, (cudaStream_t)stream,
                                       nullptr, 0, 0, 1, -1, false);
}

// Test hook: mq_launch_gemm_bf16 (no residual) whose producer never requests k-block drop_kb (0 <= drop_kb < K / 64),
// so one bounded wait of every CTA runs out: the kernel must return, set MQ_STATUS_WAIT_TIMEOUT in *status, store
// nothing, and leave the device usable.  Not used by any production path.
extern "C" int mq_debug_gemm_drop_load(const void* A, int lda, const void* B, void* C, int M, int N, int K, int ldc,
                                       unsigned int* status, void* stream, int drop_kb) {
    if (!A || !B || !C || !status || M <= 0 || N <= 0 || K <= 0 || drop_kb < 0 || drop_kb >= K / GM_BK) return MQ_ERR_BAD_ARG;
    if (lda % 8 != 0 || ldc % 8 != 0) return MQ_ERR_ALIGNMENT;
    return launch_gemm<128, EPI_STORE>((const bf16*)A, lda, (const bf16*)B, nullptr, (bf16*)C, nullptr, M, N, K, ldc, status, (cudaStream_t)stream,
                                       nullptr, 0, 0, 1, drop_kb, false);
}

static int prefill_impl(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pb, const int* ids,
                        int seq_len, int pos0, const bf16* audio, int audio_start, int audio_len, int* out_token, float* logits,
                        void* stream_v);

extern "C" int mq_launch_prefill(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pb, const int* ids,
                                 int seq_len, int pos0, int* out_token, float* logits, void* stream_v) {
    return prefill_impl(model, dbuf, pb, ids, seq_len, pos0, nullptr, 0, 0, out_token, logits, stream_v);
}

extern "C" int mq_launch_prefill_asr(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pb, const int* ids,
                                     int seq_len, int pos0, const void* audio_embeds, int audio_start, int audio_len,
                                     int* out_token, float* logits, void* stream_v) {
    if (!audio_embeds || audio_len <= 0 || audio_start < 0 || audio_start + audio_len > seq_len) return MQ_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(audio_embeds) & 15u) != 0) return MQ_ERR_ALIGNMENT;
    return prefill_impl(model, dbuf, pb, ids, seq_len, pos0, (const bf16*)audio_embeds, audio_start, audio_len, out_token, logits, stream_v);
}

static int prefill_impl(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pb, const int* ids,
                        int seq_len, int pos0, const bf16* audio, int audio_start, int audio_len, int* out_token, float* logits,
                        void* stream_v) {
    if (!model || !dbuf || !pb || !ids || !out_token) return MQ_ERR_BAD_ARG;
    if (!pb->h || !pb->x || !pb->qkv || !pb->attn || !pb->act) return MQ_ERR_BAD_ARG;
    if (seq_len <= 0 || pos0 < 0) return MQ_ERR_BAD_ARG;
    if (seq_len > pb->max_tokens || pos0 + seq_len > model->max_seq_len) return MQ_ERR_TOO_LONG;
    cudaStream_t stream = (cudaStream_t)stream_v;
    const int S = seq_len;
    bf16* h = (bf16*)pb->h; bf16* x = (bf16*)pb->x; bf16* qkv = (bf16*)pb->qkv; bf16* attn = (bf16*)pb->attn; bf16* act = (bf16*)pb->act;
    unsigned int* status = dbuf->status;
    static bool fa_attr[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const size_t fa_smem = FA_SMEM;
    if (dev >= 0 && dev < 64 && !fa_attr[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_pf_attention, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem);
        if (e != cudaSuccess) return (int)e;
        fa_attr[dev] = true;
    }
    // From 128 prompt rows on the attention runs on tcgen05, its K and V tiles straight from the cache.  The V map
    // is a stack of (layer, kv head) planes that end at the prompt's last key: what the cache holds beyond it
    // (possibly not even numbers) is multiplied by probabilities of zero and must read as zero.
    const bool use_tc = S >= TA_BQ;
    CUtensorMap map_q, map_k, map_v;
    if (use_tc) {
        static bool ta_attr[64] = {false};
        if (dev >= 0 && dev < 64 && !ta_attr[dev]) {
            cudaError_t e = cudaFuncSetAttribute(k_pf_attention_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TA_SMEM);
            if (e != cudaSuccess) return (int)e;
            ta_attr[dev] = true;
        }
        int mrc = get_map(qkv, (uint64_t)S, (uint64_t)QKV, (uint64_t)QKV, TA_BQ, &map_q);
        if (mrc == MQ_OK) mrc = get_map(dbuf->k_cache, (uint64_t)model->num_layers * NKV * model->max_seq_len, (uint64_t)D, (uint64_t)D, TA_BK, &map_k);
        if (mrc == MQ_OK)
            mrc = get_map(dbuf->v_cache, (uint64_t)(pos0 + S), (uint64_t)D, (uint64_t)D, TA_BK, &map_v, (uint64_t)model->num_layers * NKV,
                          (uint64_t)model->max_seq_len * D);
        if (mrc != MQ_OK) return mrc;
    }
    launch_pdl(k_pf_embed, dim3(S), dim3(128), 0, stream, ids, (const bf16*)model->embed, h, model->vocab_size, status, audio,
               audio_start, audio_len);
    int rc;
    const bool big = S >= 1024;
    // Between 512 and 1024 rows the N = 1024 projections (O, down) split K over two CTAs per 128 x 128 tile:
    // 64-wide tiles re-read the A operand sixteen times and are bound by L2 traffic.  The fp32 planes land in
    // the qkv buffer (free after attention; 2 x S x 1024 floats fill it exactly) and one kernel adds them to the
    // residual stream and applies the RMSNorm that follows (the next layer's input norm after the down projection).
    // Above 1024 and up to 2048 rows the same with 128 x 256 tiles (N = 256 instructions, half the A traffic per FLOP).
    const bool splitk = S >= 512 && S <= 2048 && (size_t)pb->max_tokens * QKV * sizeof(bf16) >= (size_t)2 * S * H * sizeof(float);
    const bool wide = splitk && S > 1024;
    float* part = reinterpret_cast<float*>(qkv);
    for (int l = 0; l < model->num_layers; ++l) {
        const MqLayerWeights& w = model->layers[l];
        if (l == 0 || !splitk)
            launch_pdl(k_pf_rmsnorm, dim3((S + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.input_layernorm, x, S);
        // q | k | v in one launch: 32 column tiles from three weight matrices
        // from 1024 rows on: 128 x 256 tiles (one N = 256 instruction per k-step), 256 x 256 from 2048 rows; 128 CTAs either way
        rc = S >= 2048 ? launch_gemm<256, EPI_STORE, 2>(x, H, (const bf16*)w.q_proj, (const bf16*)w.k_proj, qkv, nullptr, S, QKV, H, QKV, status, stream,
                                                        (const bf16*)w.v_proj, QSZ, KVSZ)
           : big ? launch_gemm<256, EPI_STORE, 1>(x, H, (const bf16*)w.q_proj, (const bf16*)w.k_proj, qkv, nullptr, S, QKV, H, QKV, status, stream,
                                                  (const bf16*)w.v_proj, QSZ, KVSZ)
                 : launch_gemm<128, EPI_STORE>(x, H, (const bf16*)w.q_proj, (const bf16*)w.k_proj, qkv, nullptr, S, QKV, H, QKV, status, stream,
                                               (const bf16*)w.v_proj, QSZ, KVSZ);
        if (rc) return rc;
        launch_pdl(k_pf_qknorm_rope, dim3(dim3(S, S <= 1024 ? 4 : 2)), dim3(256), 0, stream, qkv, (const bf16*)w.q_norm, (const bf16*)w.k_norm, (const bf16*)model->cos_table,
                                                         (const bf16*)model->sin_table, (bf16*)dbuf->k_cache, (bf16*)dbuf->v_cache, l, pos0,
                                                         model->max_seq_len, nullptr, 0, nullptr, 0, 0, nullptr);
        if (use_tc) {
            launch_pdl(k_pf_attention_tc, dim3(NQ, (S + TA_BQ - 1) / TA_BQ), dim3(TA_THREADS), TA_SMEM, stream, map_q, map_k, map_v, attn, S, pos0, l,
                       model->max_seq_len, status);
        } else {
            launch_pdl(k_pf_attention, dim3(dim3(NQ, (S + FA_BQ - 1) / FA_BQ)), dim3(FA_THREADS), fa_smem, stream, qkv, (const bf16*)dbuf->k_cache,
                       (const bf16*)dbuf->v_cache, attn, S, pos0, l, model->max_seq_len, PackedTiles());
        }
        // N = 1024: with M <= 1024 a 128-wide tile gives at most 64 CTAs, 64-wide tiles double that
        if (splitk) {
            rc = wide ? launch_gemm<256, EPI_PARTIAL>(attn, QSZ, (const bf16*)w.o_proj, nullptr, (bf16*)part, nullptr, S, H, QSZ, H, status, stream,
                                                      nullptr, 0, 0, 2)
                      : launch_gemm<128, EPI_PARTIAL>(attn, QSZ, (const bf16*)w.o_proj, nullptr, (bf16*)part, nullptr, S, H, QSZ, H, status, stream,
                                                      nullptr, 0, 0, 2);
            if (rc) return rc;
            launch_pdl(k_sk_resid_norm, dim3(S), dim3(256), 0, stream, (const float*)part, 2, S, h, (const bf16*)w.post_attn_layernorm, x);
        } else {
            rc = (S <= 1024) ? launch_gemm<64, EPI_RESID>(attn, QSZ, (const bf16*)w.o_proj, nullptr, h, h, S, H, QSZ, H, status, stream)
                             : launch_gemm<128, EPI_RESID>(attn, QSZ, (const bf16*)w.o_proj, nullptr, h, h, S, H, QSZ, H, status, stream);
            if (rc) return rc;
            launch_pdl(k_pf_rmsnorm, dim3((S + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.post_attn_layernorm, x, S);
        }
        // from 1024 rows on: 256 x (96 gate + 96 up) tiles, 128 CTAs at 1024 rows and two even rounds at 2048
        rc = big ? launch_gemm<96, EPI_SWIGLU, 2>(x, H, (const bf16*)w.gate_proj, (const bf16*)w.up_proj, act, nullptr, S, I, H, I, status, stream)
                 : launch_gemm<128, EPI_SWIGLU>(x, H, (const bf16*)w.gate_proj, (const bf16*)w.up_proj, act, nullptr, S, I, H, I, status, stream);
        if (rc) return rc;
        if (splitk) {
            rc = wide ? launch_gemm<256, EPI_PARTIAL>(act, I, (const bf16*)w.down_proj, nullptr, (bf16*)part, nullptr, S, H, I, H, status, stream,
                                                      nullptr, 0, 0, 2)
                      : launch_gemm<128, EPI_PARTIAL>(act, I, (const bf16*)w.down_proj, nullptr, (bf16*)part, nullptr, S, H, I, H, status, stream,
                                                      nullptr, 0, 0, 2);
            if (rc) return rc;
            const bf16* next_norm = l + 1 < model->num_layers ? (const bf16*)model->layers[l + 1].input_layernorm : nullptr;
            launch_pdl(k_sk_resid_norm, dim3(S), dim3(256), 0, stream, (const float*)part, 2, S, h, next_norm, x);
        } else {
            rc = (S <= 1024) ? launch_gemm<64, EPI_RESID>(act, I, (const bf16*)w.down_proj, nullptr, h, h, S, H, I, H, status, stream)
                             : launch_gemm<128, EPI_RESID>(act, I, (const bf16*)w.down_proj, nullptr, h, h, S, H, I, H, status, stream);
            if (rc) return rc;
        }
    }
    // last row -> decode hidden buffer, then the decode path's LM head + arg-max
    launch_pdl(k_pf_copy_row, dim3(1), dim3(H / 8), 0, stream, h + (size_t)(S - 1) * H, (bf16*)dbuf->hidden);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return launch_lmhead_only(model, dbuf, out_token, logits, stream);
}

// Prompts of several sequences packed row after row (a ragged batch in one pass): the linears
// see one matrix of total_rows rows, QK-norm/RoPE and the cache writes use the per-row tables,
// attention the per-tile tables, and the next token of every sequence comes from its last row
// through the batched LM head.  bb->positions[b] must hold len_b - 1 on entry (the arg-max kernel
// advances it to len_b).  All tables are device arrays built by the caller.
extern "C" int mq_launch_prefill_packed(const MqModel* model, const MqBatchBuffers* bb, const int* ids, const int* row_seq,
                                        const int* row_pos, const int* tile_seq, const int* tile_q0, const int* seq_len,
                                        const int* seq_row0, int total_rows, int num_tiles, int* out_tokens, void* stream_v) {
    if (!model || !bb || !ids || !row_seq || !row_pos || !tile_seq || !tile_q0 || !seq_len || !seq_row0 || !out_tokens) return MQ_ERR_BAD_ARG;
    if (!bb->k_cache || !bb->v_cache || !bb->positions || !bb->logits || !bb->status) return MQ_ERR_BAD_ARG;
    const MqPrefillBuffers* pb = &bb->act;
    if (!pb->h || !pb->x || !pb->qkv || !pb->attn || !pb->act) return MQ_ERR_BAD_ARG;
    const int B = bb->batch, T = total_rows;
    if (B <= 0 || T < B || num_tiles <= 0) return MQ_ERR_BAD_ARG;
    if (T > pb->max_tokens) return MQ_ERR_TOO_LONG;
    if (model->vocab_size % 128 != 0) return MQ_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_v;
    bf16* h = (bf16*)pb->h; bf16* x = (bf16*)pb->x; bf16* qkv = (bf16*)pb->qkv; bf16* attn = (bf16*)pb->attn; bf16* act = (bf16*)pb->act;
    unsigned int* status = bb->status;
    const size_t seq_stride = (size_t)model->num_layers * NKV * model->max_seq_len * D;
    static bool fa_attr[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !fa_attr[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_pf_attention, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_SMEM);
        if (e != cudaSuccess) return (int)e;
        fa_attr[dev] = true;
    }
    PackedTiles pt;
    pt.tile_seq = tile_seq; pt.tile_q0 = tile_q0; pt.seq_len = seq_len; pt.seq_row0 = seq_row0; pt.seq_stride = seq_stride;
    launch_pdl(k_pf_embed, dim3(T), dim3(128), 0, stream, ids, (const bf16*)model->embed, h, model->vocab_size, status,
               (const bf16*)nullptr, 0, 0);
    int rc;
    const bool big = T >= 1024;
    for (int l = 0; l < model->num_layers; ++l) {
        const MqLayerWeights& w = model->layers[l];
        launch_pdl(k_pf_rmsnorm, dim3((T + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.input_layernorm, x, T);
        rc = big ? launch_gemm<128, EPI_STORE, 2>(x, H, (const bf16*)w.q_proj, (const bf16*)w.k_proj, qkv, nullptr, T, QKV, H, QKV, status, stream,
                                                  (const bf16*)w.v_proj, QSZ, KVSZ)
                 : launch_gemm<128, EPI_STORE>(x, H, (const bf16*)w.q_proj, (const bf16*)w.k_proj, qkv, nullptr, T, QKV, H, QKV, status, stream,
                                               (const bf16*)w.v_proj, QSZ, KVSZ);
        if (rc) return rc;
        launch_pdl(k_pf_qknorm_rope, dim3(dim3(T, 1)), dim3(256), 0, stream, qkv, (const bf16*)w.q_norm, (const bf16*)w.k_norm, (const bf16*)model->cos_table,
                                                         (const bf16*)model->sin_table, (bf16*)bb->k_cache, (bf16*)bb->v_cache, l, 0,
                                                         model->max_seq_len, row_pos, seq_stride, nullptr, 0, 0, row_seq);
        launch_pdl(k_pf_attention, dim3(dim3(NQ, num_tiles)), dim3(FA_THREADS), FA_SMEM, stream, qkv, (const bf16*)bb->k_cache, (const bf16*)bb->v_cache,
                                                                       attn, 0, 0, l, model->max_seq_len, pt);
        rc = (T <= 1024) ? launch_gemm<64, EPI_RESID>(attn, QSZ, (const bf16*)w.o_proj, nullptr, h, h, T, H, QSZ, H, status, stream)
                         : launch_gemm<128, EPI_RESID>(attn, QSZ, (const bf16*)w.o_proj, nullptr, h, h, T, H, QSZ, H, status, stream);
        if (rc) return rc;
        launch_pdl(k_pf_rmsnorm, dim3((T + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.post_attn_layernorm, x, T);
        rc = big ? launch_gemm<128, EPI_SWIGLU, 2>(x, H, (const bf16*)w.gate_proj, (const bf16*)w.up_proj, act, nullptr, T, I, H, I, status, stream)
                 : launch_gemm<128, EPI_SWIGLU>(x, H, (const bf16*)w.gate_proj, (const bf16*)w.up_proj, act, nullptr, T, I, H, I, status, stream);
        if (rc) return rc;
        rc = (T <= 1024) ? launch_gemm<64, EPI_RESID>(act, I, (const bf16*)w.down_proj, nullptr, h, h, T, H, I, H, status, stream)
                         : launch_gemm<128, EPI_RESID>(act, I, (const bf16*)w.down_proj, nullptr, h, h, T, H, I, H, status, stream);
        if (rc) return rc;
    }
    // last row of every sequence -> final norm -> LM head -> arg-max (advances positions[b] to len_b)
    launch_pdl(k_pf_gather_last, dim3(B), dim3(H / 8), 0, stream, h, seq_row0, seq_len, attn);
    launch_pdl(k_pf_rmsnorm, dim3((B + 7) / 8), dim3(256), 0, stream, attn, (const bf16*)model->final_norm, x, B);
    rc = launch_gemm<128, EPI_STORE_2CTA>(x, H, (const bf16*)model->lm_head, nullptr, (bf16*)bb->logits, nullptr, B, model->vocab_size, H,
                                     model->vocab_size, status, stream);
    if (rc) return rc;
    launch_pdl(k_bd_argmax_advance, dim3(B), dim3(1024), 0, stream, (const bf16*)bb->logits, model->vocab_size, out_tokens, bb->positions, (float*)nullptr);
    return (int)cudaGetLastError();
}

// kernels of one step on the tile-GEMM path (batch > 64); the split-K path for smaller batches launches two fewer per layer
extern "C" int mq_decode_batch_launch_count(int num_layers) { return 1 + num_layers * 10 + 3; }

// How a batched attention launch is shaped for `items` = 8 x batch (sequence, kv head) pairs.  Up to one
// item per SM: twelve-warp CTAs, the keys of every item split over up to four CTAs while those still fit one
// round.  Beyond: six-warp CTAs, two per SM.  The SM streams with twelve warps either way, but two CTAs
// per SM are at different points of their items, so one CTA's ring fill and warp merge (about 4 us per
// item, during which a lone twelve-warp CTA leaves the SM's memory pipeline idle) overlap the other's
// streaming: 2.68 -> 2.49 ms per step at batch 64 / context 1024, 2.12 -> 1.90 at context 500.  The items of
// the full rounds get one CTA each and those of the last, partly empty round are split so that they
// fill it (384 items on 296 slots: 296 whole, 88 in three parts).  Splitting ALL items was measured slower
// (3.02 vs 2.68 ms per step with twelve-warp halves), four- and three-warp CTAs (three and four per SM)
// too (2.58, 2.55).  Depends on the batch size only, so a captured graph stays valid.
struct BdShape { int warps, n_full, p_tail; };
static BdShape bd_shape(int items, int sms, bool can_split) {
    if (items <= sms) {
        int p = can_split ? sms / items : 1;
        p = p > BD_MAX_PARTS ? BD_MAX_PARTS : p;
        return p < 2 ? BdShape{12, items, 1} : BdShape{12, 0, p};
    }
    const int slots = 2 * sms, rem = items % slots;
    if (!can_split || rem == 0) return {6, items, 1};
    int p = slots / rem;                                         // parts that still fit the last round
    p = p > BD_MAX_PARTS ? BD_MAX_PARTS : p;
    return p < 2 ? BdShape{6, items, 1} : BdShape{6, items - rem, p};
}

template <bool FP8, int WARPS>
static int bd_set_smem() {
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_bd_attention<FP8, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bd_smem_bytes(WARPS));
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    return MQ_OK;
}

// attention of one layer of a batched decode step, from the bf16 caches or from the e4m3 shadow caches
template <bool FP8, int WARPS>
static void launch_bd_attention_t(int B, BdShape sh, cudaStream_t stream, const bf16* qkv, const MqBatchBuffers* bb, const MqKvFp8* kv8, bf16* attn,
                                  int l, const MqModel* model, size_t seq_stride, const BdQkFuse& qk) {
    const int ctas = sh.n_full + (B * NKV - sh.n_full) * sh.p_tail;
    launch_pdl(k_bd_attention<FP8, WARPS>, dim3(ctas), dim3(WARPS * 32), bd_smem_bytes(WARPS), stream, qkv, (const bf16*)bb->k_cache,
               (const bf16*)bb->v_cache, attn, (const int*)bb->positions, l, model->max_seq_len, seq_stride,
               (uint8_t*)(kv8 ? kv8->k_fp8 : nullptr), (uint8_t*)(kv8 ? kv8->v_fp8 : nullptr), (const float*)(kv8 ? kv8->k_scale : nullptr),
               (const float*)(kv8 ? kv8->v_scale : nullptr), model->num_layers * NKV, bb->attn_parts, bb->attn_tickets, sh.n_full, sh.p_tail, qk);
}
static void launch_bd_attention(int B, BdShape sh, cudaStream_t stream, const bf16* qkv, const MqBatchBuffers* bb, const MqKvFp8* kv8, bf16* attn, int l,
                                const MqModel* model, size_t seq_stride, const BdQkFuse& qk) {
    if (kv8) {
        if (sh.warps == 6) launch_bd_attention_t<true, 6>(B, sh, stream, qkv, bb, kv8, attn, l, model, seq_stride, qk);
        else launch_bd_attention_t<true, 12>(B, sh, stream, qkv, bb, kv8, attn, l, model, seq_stride, qk);
    } else {
        if (sh.warps == 6) launch_bd_attention_t<false, 6>(B, sh, stream, qkv, bb, kv8, attn, l, model, seq_stride, qk);
        else launch_bd_attention_t<false, 12>(B, sh, stream, qkv, bb, kv8, attn, l, model, seq_stride, qk);
    }
}

static int decode_batch_impl(const MqModel* model, const MqBatchBuffers* bb, const MqKvFp8* kv8, const int* in_tokens, int* out_tokens,
                             float* logits_f32, void* stream_v) {
    if (!model || !bb || !in_tokens || !out_tokens) return MQ_ERR_BAD_ARG;
    if (kv8 && (!kv8->k_fp8 || !kv8->v_fp8 || !kv8->k_scale || !kv8->v_scale)) return MQ_ERR_BAD_ARG;
    if (!bb->k_cache || !bb->v_cache || !bb->positions || !bb->logits || !bb->status) return MQ_ERR_BAD_ARG;
    const MqPrefillBuffers* pb = &bb->act;
    if (!pb->h || !pb->x || !pb->qkv || !pb->attn || !pb->act) return MQ_ERR_BAD_ARG;
    const int B = bb->batch;
    if (B <= 0 || B > pb->max_tokens) return MQ_ERR_BAD_ARG;
    if (model->vocab_size % 128 != 0) return MQ_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_v;
    bf16* h = (bf16*)pb->h; bf16* x = (bf16*)pb->x; bf16* qkv = (bf16*)pb->qkv; bf16* attn = (bf16*)pb->attn; bf16* act = (bf16*)pb->act;
    unsigned int* status = bb->status;
    const size_t seq_stride = (size_t)model->num_layers * NKV * model->max_seq_len * D;
    int rc = bd_set_smem<false, 6>();
    if (rc == MQ_OK) rc = bd_set_smem<false, 12>();
    if (rc == MQ_OK) rc = bd_set_smem<true, 6>();
    if (rc == MQ_OK) rc = bd_set_smem<true, 12>();
    if (rc != MQ_OK) return rc;
    static int sm_count[64] = {0};
    {
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
        if (!sm_count[dev]) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        if (sm_count[dev] <= 0) return MQ_ERR_UNSUPPORTED;
    }
    int dev_now = 0;
    cudaGetDevice(&dev_now);
    const bool can_split = bb->attn_parts != nullptr && bb->attn_tickets != nullptr &&
                           bb->attn_parts_bytes >= (size_t)B * NKV * BD_MAX_PARTS * 2 * BD_PART * sizeof(float);
    const BdShape shape = bd_shape(B * NKV, sm_count[dev_now], can_split);
    launch_pdl(k_pf_embed, dim3(B), dim3(128), 0, stream, in_tokens, (const bf16*)model->embed, h, model->vocab_size, status,
               (const bf16*)nullptr, 0, 0);
    const size_t need_part = (size_t)4 * B * 2 * I * sizeof(float);   // largest partial: gate|up, 4 K-splits
    const bool skinny = B <= 64 && bb->partials != nullptr && bb->partials_bytes >= need_part;
    if (skinny) {
        float* part = bb->partials;
        launch_pdl(k_pf_rmsnorm, dim3((B + 7) / 8), dim3(256), 0, stream, h, (const bf16*)model->layers[0].input_layernorm, x, B);
        for (int l = 0; l < model->num_layers; ++l) {
            const MqLayerWeights& w = model->layers[l];
            const bf16* wqkv[3] = {(const bf16*)w.q_proj, (const bf16*)w.k_proj, (const bf16*)w.v_proj};
            const int rqkv[3] = {QSZ, KVSZ, KVSZ};
            rc = launch_skinny(wqkv, rqkv, 3, x, H, part, B, H, 4, status, stream);
            if (rc) return rc;
            // the attention CTAs sum the four K-split planes of their heads, apply QK-norm + RoPE and write the new K / V rows
            const BdQkFuse qk{(const float*)part, 4, B, (const bf16*)w.q_norm, (const bf16*)w.k_norm, (const bf16*)model->cos_table,
                              (const bf16*)model->sin_table};
            launch_bd_attention(B, shape, stream, qkv, bb, kv8, attn, l, model, seq_stride, qk);
            const bf16* wo[1] = {(const bf16*)w.o_proj};
            const int ro[1] = {H};
            rc = launch_skinny(wo, ro, 1, attn, QSZ, part, B, QSZ, 8, status, stream);
            if (rc) return rc;
            launch_pdl(k_sk_resid_norm, dim3(B), dim3(256), 0, stream, part, 8, B, h, (const bf16*)w.post_attn_layernorm, x);
            const bf16* wgu[2] = {(const bf16*)w.gate_proj, (const bf16*)w.up_proj};
            const int rgu[2] = {I, I};
            rc = launch_skinny(wgu, rgu, 2, x, H, part, B, H, 4, status, stream);
            if (rc) return rc;
            launch_pdl(k_sk_swiglu, dim3((B * I + 255) / 256), dim3(256), 0, stream, part, 4, B, act);
            const bf16* wd[1] = {(const bf16*)w.down_proj};
            rc = launch_skinny(wd, ro, 1, act, I, part, B, I, 8, status, stream);
            if (rc) return rc;
            const bf16* next_norm = (l + 1 < model->num_layers) ? (const bf16*)model->layers[l + 1].input_layernorm : (const bf16*)model->final_norm;
            launch_pdl(k_sk_resid_norm, dim3(B), dim3(256), 0, stream, part, 8, B, h, next_norm, x);
        }
    } else {
    for (int l = 0; l < model->num_layers; ++l) {
        const MqLayerWeights& w = model->layers[l];
        launch_pdl(k_pf_rmsnorm, dim3((B + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.input_layernorm, x, B);
        rc = launch_gemm<128, EPI_STORE>(x, H, (const bf16*)w.q_proj, nullptr, qkv, nullptr, B, QSZ, H, QKV, status, stream);
        if (rc) return rc;
        rc = launch_gemm<128, EPI_STORE>(x, H, (const bf16*)w.k_proj, nullptr, qkv + QSZ, nullptr, B, KVSZ, H, QKV, status, stream);
        if (rc) return rc;
        rc = launch_gemm<128, EPI_STORE>(x, H, (const bf16*)w.v_proj, nullptr, qkv + QSZ + KVSZ, nullptr, B, KVSZ, H, QKV, status, stream);
        if (rc) return rc;
        launch_pdl(k_pf_qknorm_rope, dim3(dim3(B, 4)), dim3(256), 0, stream, qkv, (const bf16*)w.q_norm, (const bf16*)w.k_norm, (const bf16*)model->cos_table,
                                                         (const bf16*)model->sin_table, (bf16*)bb->k_cache, (bf16*)bb->v_cache, l, 0,
                                                         model->max_seq_len, bb->positions, seq_stride, nullptr, 0, 0, nullptr);
        launch_bd_attention(B, shape, stream, qkv, bb, kv8, attn, l, model, seq_stride, BdQkFuse{});
        rc = launch_gemm<128, EPI_RESID>(attn, QSZ, (const bf16*)w.o_proj, nullptr, h, h, B, H, QSZ, H, status, stream);
        if (rc) return rc;
        launch_pdl(k_pf_rmsnorm, dim3((B + 7) / 8), dim3(256), 0, stream, h, (const bf16*)w.post_attn_layernorm, x, B);
        rc = launch_gemm<128, EPI_SWIGLU>(x, H, (const bf16*)w.gate_proj, (const bf16*)w.up_proj, act, nullptr, B, I, H, I, status, stream);
        if (rc) return rc;
        rc = launch_gemm<128, EPI_RESID>(act, I, (const bf16*)w.down_proj, nullptr, h, h, B, H, I, H, status, stream);
        if (rc) return rc;
    }
    launch_pdl(k_pf_rmsnorm, dim3((B + 7) / 8), dim3(256), 0, stream, h, (const bf16*)model->final_norm, x, B);
    }
    rc = launch_gemm<128, EPI_STORE_2CTA>(x, H, (const bf16*)model->lm_head, nullptr, (bf16*)bb->logits, nullptr, B, model->vocab_size, H,
                                     model->vocab_size, status, stream);
    if (rc) return rc;
    launch_pdl(k_bd_argmax_advance, dim3(B), dim3(1024), 0, stream, (const bf16*)bb->logits, model->vocab_size, out_tokens, bb->positions, logits_f32);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_decode_batch(const MqModel* model, const MqBatchBuffers* bb, const int* in_tokens, int* out_tokens,
                                      float* logits_f32, void* stream_v) {
    return decode_batch_impl(model, bb, nullptr, in_tokens, out_tokens, logits_f32, stream_v);
}

extern "C" int mq_launch_decode_batch_kv8(const MqModel* model, const MqBatchBuffers* bb, const MqKvFp8* kv8, const int* in_tokens,
                                          int* out_tokens, float* logits_f32, void* stream_v) {
    if (!kv8) return MQ_ERR_BAD_ARG;
    return decode_batch_impl(model, bb, kv8, in_tokens, out_tokens, logits_f32, stream_v);
}

// ---------------------------------------------------------------- FP8 shadow cache
// One CTA per (layer, kv head): scale = max |x| over positions [start, end) / 448 (1 for an all-zero
// span), then every element of the span as e4m3(x / scale), K and V separately (reference:
// split_quantize_kv_cache_fp8_kernel, csrc/megakernel/split_decode_gemm.cu:223-300).
__global__ void __launch_bounds__(256) k_kv_quantize_fp8(const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                                         uint8_t* __restrict__ k8, uint8_t* __restrict__ v8, float* __restrict__ k_scale,
                                                         float* __restrict__ v_scale, int max_seq, int start, int end) {
    __shared__ float s_k[8], s_v[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t base = (size_t)blockIdx.x * max_seq * D;
    const int n8 = (end - start) * (D / 8);                        // 16-byte groups of the span
    const uint4* kp = reinterpret_cast<const uint4*>(k_cache + base + (size_t)start * D);
    const uint4* vp = reinterpret_cast<const uint4*>(v_cache + base + (size_t)start * D);
    auto amax4 = [](const uint4& u) {
        float m = fmaxf(fabsf(bf_lo(u.x)), fabsf(bf_hi(u.x)));
        m = fmaxf(m, fmaxf(fabsf(bf_lo(u.y)), fabsf(bf_hi(u.y))));
        m = fmaxf(m, fmaxf(fabsf(bf_lo(u.z)), fabsf(bf_hi(u.z))));
        return fmaxf(m, fmaxf(fabsf(bf_lo(u.w)), fabsf(bf_hi(u.w))));
    };
    float km = 0.f, vm = 0.f;
    for (int i = tid; i < n8; i += 256) {
        km = fmaxf(km, amax4(kp[i]));
        vm = fmaxf(vm, amax4(vp[i]));
    }
    km = warp_max(km);
    vm = warp_max(vm);
    if (lane == 0) { s_k[warp] = km; s_v[warp] = vm; }
    __syncthreads();
    km = 0.f; vm = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { km = fmaxf(km, s_k[w]); vm = fmaxf(vm, s_v[w]); }
    const float ks = kv_fp8_scale_of(km), vs = kv_fp8_scale_of(vm);
    if (tid == 0) { k_scale[blockIdx.x] = ks; v_scale[blockIdx.x] = vs; }
    const float ik = 1.0f / ks, iv = 1.0f / vs;
    uint2* k8p = reinterpret_cast<uint2*>(k8 + base + (size_t)start * D);
    uint2* v8p = reinterpret_cast<uint2*>(v8 + base + (size_t)start * D);
    for (int i = tid; i < n8; i += 256) {
        const uint4 a = kp[i], b = vp[i];
        k8p[i] = make_uint2(f32x4_to_fp8x4(bf_lo(a.x) * ik, bf_hi(a.x) * ik, bf_lo(a.y) * ik, bf_hi(a.y) * ik),
                            f32x4_to_fp8x4(bf_lo(a.z) * ik, bf_hi(a.z) * ik, bf_lo(a.w) * ik, bf_hi(a.w) * ik));
        v8p[i] = make_uint2(f32x4_to_fp8x4(bf_lo(b.x) * iv, bf_hi(b.x) * iv, bf_lo(b.y) * iv, bf_hi(b.y) * iv),
                            f32x4_to_fp8x4(bf_lo(b.z) * iv, bf_hi(b.z) * iv, bf_lo(b.w) * iv, bf_hi(b.w) * iv));
    }
}

extern "C" int mq_launch_kv_quantize_fp8(const void* k_cache, const void* v_cache, const MqKvFp8* kv8, int num_layers, int max_seq_len,
                                         int start_pos, int end_pos, void* stream_v) {
    if (!k_cache || !v_cache || !kv8 || !kv8->k_fp8 || !kv8->v_fp8 || !kv8->k_scale || !kv8->v_scale) return MQ_ERR_BAD_ARG;
    if (num_layers <= 0 || max_seq_len <= 0) return MQ_ERR_BAD_ARG;
    const int start = start_pos < 0 ? 0 : start_pos, end = end_pos > max_seq_len ? max_seq_len : end_pos;
    if (start >= end) return MQ_OK;                                  // an empty span is a no-op, as in the reference
    k_kv_quantize_fp8<<<num_layers * NKV, 256, 0, (cudaStream_t)stream_v>>>((const bf16*)k_cache, (const bf16*)v_cache, (uint8_t*)kv8->k_fp8,
                                                                            (uint8_t*)kv8->v_fp8, kv8->k_scale, kv8->v_scale, max_seq_len, start, end);
    return (int)cudaGetLastError();
}
