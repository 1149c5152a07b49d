// Persistent batch-1 greedy decode for sm_100a: ONE cooperative launch of one CTA per SM
// runs n_steps decode steps (all layers, LM head, arg-max, next embedding).  It replaces the
// reference's cooperative megakernel and its device-resident chains
// (csrc/megakernel/fused_decode_ldg_kernel.inl:43-258, bindings_prefill.cpp:1045-1349).
//
// A decode step is HBM-bound (1.19 GB of bf16 weights per token) but is a chain of ~140
// dependent phases, so the design separates the two:
//
//  * Weights never depend on activations.  At load time they are repacked into one
//    contiguous byte stream per WARP (8 per CTA), in exactly the order that warp consumes them
//    and already in the register layout of the mma.sync A operand.  Each warp streams its own
//    bytes through a private ring of 2 KB shared-memory slots with 1-D TMA bulk copies (no
//    multicast): it waits for a slot, multiplies, and refills the slot it has just used with
//    the unit nine places ahead.  There is no producer warp and no hand-shake between warps;
//    the stream runs ahead of the arithmetic by the ring's size (144 KB per SM) across phase,
//    layer and step boundaries.  The LM head (tied embedding, tiled the same way) is the tail
//    of every step's stream.
//  * Activations are exchanged between CTAs through small global buffers of 32-bit words that
//    hold a bf16 value in the high half and a 16-bit phase tag in the low half: a consumer
//    re-reads its words until the tags match, so data and readiness arrive in one L2 round
//    trip and there is no flag, fence, grid barrier or kernel boundary on the critical path
//    (the reference: 225 grid.sync() per token).  fp32 split-KV partials and the arg-max keys
//    travel as 64-bit words (tag32 | payload32).
//  * Every GEMV is K-split over the CTA's eight warps (warp w owns columns w K/8 .. of every
//    row of the CTA), accumulates with mma.sync.m16n8k16 (bf16 in, fp32 out; the activation
//    vector replicated over the eight B columns) and is summed across warps in a fixed order:
//    results are bit-reproducible.  In the LM head a warp owns whole 16-row tiles instead.
//  * The layer loop runs thousands of times and must stay in the instruction cache: loops are
//    rolled, the GEMV code exists once, rare paths are out of line.
//
// Work split (planned on the host for the device's SM count): the 4096 q|k|v rows, the 3072
// gate/up row pairs and the 1024 rows of Wo / Wd are dealt out in groups of 8 rows so that every
// CTA streams the same number of bytes per layer (13 x 16 KB on 148 SMs); a CTA owns the same
// rows of Wo and Wd, which keeps the residual stream of those rows in a register.  Attention of
// kv head g runs on CTAs g, g + 8, ..: one CTA up to 128 cached positions, up to 18 splits of
// at most 128 positions beyond (context <= 2304), merged by the CTAs of splits 0 and 1.
//
// Rounding points are those of the HuggingFace bf16 model, as in decode.cu.  Every wait
// (mbarrier or tag poll) is bounded; on expiry the sticky status bit is set, later waits give
// up at once and the kernel drains.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "mq_device.cuh"

namespace mq {

#ifndef MQ_ST_WARPS
#define MQ_ST_WARPS 8
#endif
// Eight warps measured faster than sixteen (421 vs 471 us per token at context 1): a GEMV stage is
// bound by its block barriers, the partial-sum reduction and the publishing, not by the two to
// six units a warp multiplies in it, and all of those cost more with 512 threads.
constexpr int ST_WARPS = MQ_ST_WARPS;            // every warp streams and multiplies its own columns
constexpr int ST_THREADS = ST_WARPS * 32;
constexpr int ST_VT = 256;                       // threads 0..255 (warps 0..7) also do the vector work: norms, attention, publishing
constexpr int ST_VW = ST_VT / 32;
constexpr uint32_t ST_UNIT = 2048;               // bytes per ring slot = one bulk copy = 4 blocks of 512 bytes
#ifndef MQ_ST_NSLOT
#define MQ_ST_NSLOT 4
#endif
constexpr int ST_NSLOT = MQ_ST_NSLOT;            // ring slots per warp
#ifndef MQ_ST_COPY
#define MQ_ST_COPY 2
#endif
constexpr int ST_COPY = MQ_ST_COPY;              // units per bulk copy = per ring slot
constexpr uint32_t ST_SLOT_BYTES = ST_COPY * ST_UNIT;
constexpr int ST_KV_CAP = 128;                   // cached positions one CTA attends over
constexpr int ST_KV_LD = D + 8;                  // K/V rows padded by 16 bytes (conflict-free ldmatrix)
constexpr int ST_MAX_SPLIT = 18;                 // CTAs per kv head
constexpr int ST_MAX_TILES = 7;                  // 16-row tiles per GEMV phase and CTA
constexpr int ST_RED_ROWS = 16 * ST_MAX_TILES;
constexpr int ST_MIN_GRID = 128;
constexpr int ST_MAX_GRID = 256;
constexpr int ST_PART = D + 2;                   // m, l, acc[128]
constexpr int ST_STAGES = 16;                    // stage counters per (CTA, layer)
constexpr int ST_LM_TILE_UNITS = 16;             // one 16-row tile of the LM head: 64 k-steps = 32 KB

// Per-CTA plan, written by the host when the weights are packed.
struct StPlan {
    int a_row0, a_ng;          // rows of [Wq;Wk;Wv]: first row (multiple of 8) and number of 8-row groups
    int od_row0, od_ng;        // rows of Wo and Wd
    int gu_row0, gu_np;        // rows of Wg / Wu: first row and number of (8 gate + 8 up) tiles
    int lm_row0, lm_nt;        // LM head: first vocabulary row and number of 16-row tiles
    uint32_t layer_units;      // unused (the units per layer differ from warp to warp: st_layer_units)
    uint32_t pad_[3];
    unsigned long long stream_off;   // byte offset of this CTA's streams (warp 0 first) in the packed buffer
    unsigned long long pad2_;
};
static_assert(sizeof(StPlan) == 64, "plan layout");

// Units of warp w in one phase of ng 8-row groups over K columns.  A full tile (16 rows) is split by
// columns: warp w multiplies columns [w K / W, (w + 1) K / W), K / (64 W) units.  The half tile (8 rows,
// the last group of an odd count) is K / 128 units of 128 columns: warp w takes units w, w + W, ..
__host__ __device__ constexpr uint32_t st_half_units(int K, int w) { return (uint32_t)((K / 128 > w) ? (K / 128 - w + ST_WARPS - 1) / ST_WARPS : 0); }
__host__ __device__ constexpr uint32_t st_phase_units(int K, int ng, int w) {
    return (uint32_t)((ng >> 1) * (K / (64 * ST_WARPS))) + ((ng & 1) ? st_half_units(K, w) : 0u);
}
static_assert(H % (64 * ST_WARPS) == 0 && QSZ % (64 * ST_WARPS) == 0 && I % (64 * ST_WARPS) == 0, "column split of a full tile");
__host__ __device__ inline uint32_t st_layer_units(const StPlan& p, int w) {
    return st_phase_units(H, p.a_ng, w) + st_phase_units(QSZ, p.od_ng, w) + st_phase_units(H, 2 * p.gu_np, w) + st_phase_units(I, p.od_ng, w);
}
// LM tiles of warp w: tiles w, w + 8, .. of the CTA's lm_nt tiles
__host__ __device__ inline uint32_t st_lm_tiles(const StPlan& p, int w) { return p.lm_nt > w ? (uint32_t)(p.lm_nt - w + ST_WARPS - 1) / ST_WARPS : 0u; }
__host__ __device__ inline uint32_t st_step_units(const StPlan& p, int w, int num_layers) {
    return (uint32_t)num_layers * st_layer_units(p, w) + st_lm_tiles(p, w) * ST_LM_TILE_UNITS;
}

// Scratch (caller-owned, zeroed once): tagged exchange vectors, split-KV partials, arg-max keys
// and the phase counter that keeps tags unique from launch to launch.
constexpr size_t SC_XH = 0;                                    // u32 [1024]
constexpr size_t SC_XQKV = SC_XH + (size_t)H * 4;              // u32 [4096]
constexpr size_t SC_XATTN = SC_XQKV + (size_t)QKV * 4;         // u32 [2048]
constexpr size_t SC_XH1 = SC_XATTN + (size_t)QSZ * 4;          // u32 [1024]
constexpr size_t SC_XACT = SC_XH1 + (size_t)H * 4;             // u32 [3072]
constexpr size_t SC_XPART = SC_XACT + (size_t)I * 4;           // u64 [8][18][2][130]
constexpr size_t SC_XLM = SC_XPART + (size_t)NKV * ST_MAX_SPLIT * 2 * ST_PART * 8;   // u64 [2 * ST_MAX_GRID]
constexpr size_t SC_EPOCH = SC_XLM + (size_t)2 * ST_MAX_GRID * 8;                    // u32 [1]
constexpr size_t SC_BYTES = SC_EPOCH + 256;

struct StreamArgs {
    const uint8_t* packed;          // header (plans, norm vectors) + per-CTA streams
    const StPlan* plans;
    const bf16* norms;              // [num_layers][input_ln 1024 | post_ln 1024 | q_norm 128 | k_norm 128]
    const bf16* embed;
    const bf16* final_norm;
    const bf16* cos;
    const bf16* sin;
    bf16* k_cache;
    bf16* v_cache;
    uint8_t* scratch;
    unsigned int* status;
    const int* first_token;
    const int* pos0;
    const int* forced;              // optional [n_steps]: step i consumes forced[i] instead of the previous arg-max
    int* tokens_out;                // [n_steps]
    float* logits;                  // optional fp32: [n_steps][vocab] (logits_all) or [vocab] of the last step
    unsigned long long* dbg;        // optional [grid][num_layers + 1][ST_STAGES] cycle counters
    int num_layers;
    int vocab;
    int max_seq;
    int n_steps;
    int logits_all;
    int max_split;                  // min(18, grid / 8)
};


constexpr int NORM_STRIDE = 2 * H + 2 * D;

// ------------------------------------------------------------------ tagged exchange
__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// v must be exactly representable in bf16
__device__ __forceinline__ void publish(uint32_t* dst, int idx, float v, uint32_t tag16) {
    st_relaxed_u32(dst + idx, (__float_as_uint(v) & 0xffff0000u) | tag16);
}
__device__ __forceinline__ void publish_u32(unsigned long long* dst, size_t idx, uint32_t payload, uint32_t tag32) {
    st_relaxed_u64(dst + idx, ((unsigned long long)tag32 << 32) | (unsigned long long)payload);
}

constexpr long long POLL_LIMIT_CYCLES = 400000000LL;   // about 0.2 s

struct Poller {
    unsigned int* status;
    bool aborted;       // the kernel is draining
    __device__ __forceinline__ void refresh() { aborted = (ld_relaxed_u32(status) & MQ_STATUS_WAIT_TIMEOUT) != 0; }
    __device__ __forceinline__ void expire() {
        atomicOr(status, MQ_STATUS_WAIT_TIMEOUT);
        aborted = true;
    }
    static __device__ __forceinline__ bool tags_ok(const uint4& u, uint32_t tag16) {
        return ((u.x & 0xffffu) == tag16) & ((u.y & 0xffffu) == tag16) & ((u.z & 0xffffu) == tag16) & ((u.w & 0xffffu) == tag16);
    }
    // re-read four consecutive tagged words until all carry tag16 (or the kernel is draining)
    __device__ __noinline__ uint4 spin4(const uint32_t* p, uint32_t tag16) {
        uint4 v = ld_relaxed_v4(p);
        if (aborted) return v;
        const long long t0 = clock64();
        int it = 0;
        while (!tags_ok(v, tag16)) {
            if ((++it & 63) == 0) {
                refresh();
                if (aborted) return v;
                if (clock64() - t0 > POLL_LIMIT_CYCLES) { expire(); return v; }
            }
            v = ld_relaxed_v4(p);
        }
        return v;
    }
    __device__ __noinline__ uint32_t spin64(const unsigned long long* p, uint32_t tag32) {
        unsigned long long v = ld_relaxed_u64(p);
        if (aborted) return (uint32_t)v;
        const long long t0 = clock64();
        int it = 0;
        while ((uint32_t)(v >> 32) != tag32) {
            if ((++it & 63) == 0) {
                refresh();
                if (aborted) break;
                if (clock64() - t0 > POLL_LIMIT_CYCLES) { expire(); break; }
            }
            v = ld_relaxed_u64(p);
        }
        return (uint32_t)v;
    }
    __device__ __forceinline__ uint4 words4(const uint32_t* p, uint32_t tag16) {
        const uint4 v = ld_relaxed_v4(p);
        return tags_ok(v, tag16) ? v : spin4(p, tag16);
    }
    __device__ __forceinline__ float f32(const unsigned long long* p, uint32_t tag32) {
        const unsigned long long v = ld_relaxed_u64(p);
        return __uint_as_float(((uint32_t)(v >> 32) == tag32) ? (uint32_t)v : spin64(p, tag32));
    }
};

__device__ __forceinline__ void consumer_bar() { __syncthreads(); }

__device__ __forceinline__ uint2 tagged_to_bf16x4(const uint4& v) {
    uint2 o;
    o.x = (v.x >> 16) | (v.y & 0xffff0000u);
    o.y = (v.z >> 16) | (v.w & 0xffff0000u);
    return o;
}

// Warp `warp` gathers the columns of ITS half-tile units (128 columns each: units warp, warp + W, ..) of a
// tagged vector of K words, which is all its share of a K-split GEMV needs: no block barrier, and the
// warp starts as soon as its own words are in.  All loads are issued before the first tag check.
template <int K>
__device__ __forceinline__ void poll_units(Poller& po, const uint32_t* src, uint32_t tag16, bf16* dst, int warp, int lane) {
    constexpr int NU = (K / 128 + ST_WARPS - 1) / ST_WARPS;
    uint4 v[NU];
#pragma unroll
    for (int k = 0; k < NU; ++k) {
        const int u = warp + k * ST_WARPS;
        if (u < K / 128) v[k] = ld_relaxed_v4(src + u * 128 + lane * 4);
    }
#pragma unroll
    for (int k = 0; k < NU; ++k) {
        const int u = warp + k * ST_WARPS;
        if (u < K / 128) {
            if (!Poller::tags_ok(v[k], tag16)) v[k] = po.spin4(src + u * 128 + lane * 4, tag16);
            *reinterpret_cast<uint2*>(dst + u * 128 + lane * 4) = tagged_to_bf16x4(v[k]);
        }
    }
    __syncwarp();
}

__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t saddr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(saddr));
    return v;
}

// ------------------------------------------------------------------ the ring of one warp
// Slot k of the warp holds unit u with u % ST_NSLOT == k of the warp's stream.  The warp waits
// for the slot's mbarrier (completed by the bulk copy), reads the unit, and lane 0 refills the
// same slot with unit u + ST_NSLOT.  Refill and use are ordered by the warp's own program
// order, so there is no "empty" barrier.
__device__ __noinline__ void mbar_wait_slow(uint64_t* bar, uint32_t parity, unsigned int* status) { mbar_wait(bar, parity, status); }

__device__ __forceinline__ void bulk_g2s_addr(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t bar_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}

struct WRing {
    uint32_t base;            // shared address of this warp's slot 0
    uint64_t* full;           // this warp's ST_NSLOT barriers
    const uint8_t* src;       // this warp's stream (one step's worth, re-read every step)
    unsigned int* status;
    uint32_t slot;            // slot of the next unit to use
    uint32_t parity;          // its barrier phase
    uint32_t sub;             // unit within the slot
    uint32_t cur_n;           // units the slot holds
    uint32_t cidx;            // index (within a step) of the next unit to use
    uint32_t fidx;            // index (within a step) of the next unit to fetch
    uint32_t step_units;      // units per step
    uint32_t left;            // units still to fetch in this launch

    // one bulk copy of up to ST_COPY consecutive units (never across the end of a step's stream)
    __device__ __forceinline__ void fetch(uint32_t k, int lane) {
        const uint32_t n = min((uint32_t)ST_COPY, step_units - fidx);
        if (lane == 0) {
            const uint32_t bar = smem_u32(&full[k]);
            mbar_expect_tx_addr(bar, n * ST_UNIT);
            bulk_g2s_addr(base + k * ST_SLOT_BYTES, src + (size_t)fidx * ST_UNIT, n * ST_UNIT, bar);
        }
        left -= n;
        fidx += n;
        if (fidx == step_units) fidx = 0u;
    }
    // shared address of the next unit, once it has landed
    __device__ __forceinline__ uint32_t acquire() {
        if (sub == 0u) {
            if (!mbar_try_wait(&full[slot], parity)) mbar_wait_slow(&full[slot], parity, status);
            cur_n = min((uint32_t)ST_COPY, step_units - cidx);
        }
        return base + slot * ST_SLOT_BYTES + sub * ST_UNIT;
    }
    // the unit's bytes are in registers (their consumers have been issued); after the last unit
    // of a slot the slot is refilled
    __device__ __forceinline__ void release(int lane) {
        if (++cidx == step_units) cidx = 0u;
        if (++sub == cur_n) {
            sub = 0u;
            __syncwarp();
            if (left) fetch(slot, lane);
            if (++slot == (uint32_t)ST_NSLOT) { slot = 0u; parity ^= 1u; }
        }
    }
};

// ------------------------------------------------------------------ GEMV on the packed stream
// One phase = `ntf` full tiles (16 rows) and `nh` (0/1) half tile (8 rows).  Of a full tile warp w
// multiplies columns [w K / W, (w + 1) K / W) with its slice of the activation vector (bf16, shared
// memory); of the half tile the 128-column units w, w + W, ..  Stream of the warp: per full tile
// K / (64 W) units, then its units of the half tile.  A unit is four 512-byte blocks, 16 bytes per lane and block:
//   full tile, block s = k-step s of the unit (columns c = C0 + 16 tig + 4 s):
//       W[g][c, c+1] | W[g+8][c, c+1] | W[g][c+2, c+3] | W[g+8][c+2, c+3]      (a0 a1 a2 a3)
//   half tile, block u = k-steps 2u, 2u+1 (columns c = C0 + 32 tig + 8 u):
//       W[g][c .. c+7]                                  (k-step 2u: c..c+3, k-step 2u+1: c+4..c+7)
// with g = lane / 4, tig = lane % 4: a lane's B fragments of a unit are 32 (64) contiguous
// bytes of the activation vector.  Lanes 0, 4, .., 28 end with row g in c[0] and row g + 8 in
// c[2], written to red[warp][row].
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// one unit of a full tile: four k-steps into four independent accumulators
__device__ __forceinline__ void full_unit(WRing& rg, float (&c)[4][4], uint32_t xaddr, int lane) {
    const uint32_t sa = rg.acquire() + (uint32_t)lane * 16u;
    const uint4 a0 = lds128(sa), a1 = lds128(sa + 512u), a2 = lds128(sa + 1024u), a3 = lds128(sa + 1536u);
    const uint4 x0 = lds128(xaddr), x1 = lds128(xaddr + 16u);
    {
        mma_bf16(c[0], a0.x, a0.y, a0.z, a0.w, x0.x, x0.y);
        mma_bf16(c[1], a1.x, a1.y, a1.z, a1.w, x0.z, x0.w);
        mma_bf16(c[2], a2.x, a2.y, a2.z, a2.w, x1.x, x1.y);
        mma_bf16(c[3], a3.x, a3.y, a3.z, a3.w, x1.z, x1.w);
    }
    rg.release(lane);
}

__device__ __forceinline__ void gemv_phase(WRing& rg, int ntf, int nh, int K, uint32_t xs_addr, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cpw = K / ST_WARPS;                                        // this warp's columns of a full tile
    float* rw = red + warp * ST_RED_ROWS + (lane >> 2);
#pragma unroll 1
    for (int t = 0; t < ntf; ++t) {
        float c[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
        const uint32_t xl = xs_addr + (uint32_t)(warp * cpw) * 2u + (uint32_t)(lane & 3) * 32u;
#pragma unroll 1
        for (int i = 0; i < cpw; i += 64) full_unit(rg, c, xl + (uint32_t)i * 2u, lane);
        if ((lane & 3) == 0) {
            rw[t * 16] = (c[0][0] + c[1][0]) + (c[2][0] + c[3][0]);
            rw[t * 16 + 8] = (c[0][2] + c[1][2]) + (c[2][2] + c[3][2]);
        }
    }
    if (nh) {
        float c[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
        const bool odd = ((lane >> 2) & 1) != 0;
#pragma unroll 1
        for (int u = warp; u < K / 128; u += ST_WARPS) {
            const uint32_t sa = rg.acquire() + (uint32_t)lane * 16u;
            const uint4 a0 = lds128(sa), a1 = lds128(sa + 512u), a2 = lds128(sa + 1024u), a3 = lds128(sa + 1536u);
            const uint32_t xa = xs_addr + (uint32_t)u * 256u + (uint32_t)(lane & 3) * 64u;
            const uint4 x0 = lds128(xa), x1 = lds128(xa + 16u), x2 = lds128(xa + 32u), x3 = lds128(xa + 48u);
            {
                // One mma per block: rows 0-7 of the A tile are the 8 weight rows at k-step 2u, rows
                // 8-15 the SAME weight rows at k-step 2u+1; B column 0 carries the vector slice of
                // k-step 2u, column 1 that of 2u+1 (the other columns are ignored).  The row sums are
                // C[r][0] + C[r+8][1], i.e. c[0] + c[3] of lanes 0, 4, .., 28.
                mma_bf16(c[0], a0.x, a0.z, a0.y, a0.w, odd ? x0.z : x0.x, odd ? x0.w : x0.y);
                mma_bf16(c[1], a1.x, a1.z, a1.y, a1.w, odd ? x1.z : x1.x, odd ? x1.w : x1.y);
                mma_bf16(c[2], a2.x, a2.z, a2.y, a2.w, odd ? x2.z : x2.x, odd ? x2.w : x2.y);
                mma_bf16(c[3], a3.x, a3.z, a3.y, a3.w, odd ? x3.z : x3.x, odd ? x3.w : x3.y);
            }
            rg.release(lane);
        }
        // a warp without a unit of the half tile contributes zeros
        if ((lane & 3) == 0) rw[ntf * 16] = ((c[0][0] + c[0][3]) + (c[1][0] + c[1][3])) + ((c[2][0] + c[2][3]) + (c[3][0] + c[3][3]));
    }
}

// per-head RMSNorm + RoPE of a raw head held in shared memory (bf16[128]); lane owns elements
// 2 lane, 2 lane + 1 of the first half and the same of the second half
__device__ __forceinline__ void norm_rope_smem(const bf16* raw, const bf16* wn, const bf16* cosr, const bf16* sinr, int lane,
                                               float (&lo)[2], float (&hi)[2]) {
    const uint32_t ulo = *reinterpret_cast<const uint32_t*>(raw + 2 * lane), uhi = *reinterpret_cast<const uint32_t*>(raw + 64 + 2 * lane);
    const float xl[2] = {bf_lo(ulo), bf_hi(ulo)}, xh[2] = {bf_lo(uhi), bf_hi(uhi)};
    float ss = xl[0] * xl[0] + xl[1] * xl[1] + xh[0] * xh[0] + xh[1] * xh[1];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
    const uint32_t wl = *reinterpret_cast<const uint32_t*>(wn + 2 * lane), wh = *reinterpret_cast<const uint32_t*>(wn + 64 + 2 * lane);
    const uint32_t cl = *reinterpret_cast<const uint32_t*>(cosr + 2 * lane), chh = *reinterpret_cast<const uint32_t*>(cosr + 64 + 2 * lane);
    const uint32_t sl = *reinterpret_cast<const uint32_t*>(sinr + 2 * lane), sh = *reinterpret_cast<const uint32_t*>(sinr + 64 + 2 * lane);
    const float wlo[2] = {bf_lo(wl), bf_hi(wl)}, whi[2] = {bf_lo(wh), bf_hi(wh)};
    const float clo[2] = {bf_lo(cl), bf_hi(cl)}, chi[2] = {bf_lo(chh), bf_hi(chh)};
    const float slo[2] = {bf_lo(sl), bf_hi(sl)}, shi[2] = {bf_lo(sh), bf_hi(sh)};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const float nl = rbf(wlo[e] * rbf(xl[e] * r));
        const float nh = rbf(whi[e] * rbf(xh[e] * r));
        // x * cos + rotate_half(x) * sin, rotate_half = (-second half, first half)
        lo[e] = rbf(rbf(nl * clo[e]) + rbf(-nh * slo[e]));
        hi[e] = rbf(rbf(nh * chi[e]) + rbf(nl * shi[e]));
    }
}

// How the cached positions of one kv head are dealt to its CTAs at a given context length.
struct AttPlan {
    int n_act, chunk, c0, n, n_cached;
    bool active, is_last;
};
__device__ __forceinline__ AttPlan att_plan(int cta, int pos, int max_split) {
    AttPlan p;
    const int len = pos + 1;
    if (len <= ST_KV_CAP) {
        p.n_act = 1;
        p.chunk = ST_KV_CAP;
    } else {
        const int want = min(max_split, (len + 63) / 64);
        p.chunk = (((len + want - 1) / want) + 15) & ~15;
        p.n_act = (len + p.chunk - 1) / p.chunk;
    }
    const int s = cta / NKV;
    p.active = cta < NKV * max_split && s < p.n_act && p.chunk <= ST_KV_CAP;
    p.c0 = s * p.chunk;
    p.n = p.active ? min(len, p.c0 + p.chunk) - p.c0 : 0;
    p.is_last = p.active && s == p.n_act - 1;
    p.n_cached = p.is_last ? p.n - 1 : p.n;
    return p;
}

__device__ __forceinline__ unsigned long long argmax_key64(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(ST_THREADS, 1) k_decode_stream(StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* ring = smem_raw;                                                    // [ST_WARPS][ST_NSLOT][ST_UNIT]
    bf16* kt = reinterpret_cast<bf16*>(smem_raw + (size_t)ST_WARPS * ST_NSLOT * ST_SLOT_BYTES);   // [ST_KV_CAP][ST_KV_LD]
    bf16* vt = kt + (size_t)ST_KV_CAP * ST_KV_LD;
    bf16* xs = vt + (size_t)ST_KV_CAP * ST_KV_LD;                                // [3072] activation vector of a GEMV phase
    float* red = reinterpret_cast<float*>(xs + I);                               // [ST_WARPS][ST_RED_ROWS] per-warp partial sums
    float* wacc = reinterpret_cast<float*>(xs);                                  // [8][2][128], attention only (over xs + red)
    bf16* raw = reinterpret_cast<bf16*>(red + ST_WARPS * ST_RED_ROWS);           // [4][128] raw q(2g) | q(2g+1) | k | v
    bf16* qs = raw + 4 * D;                                                      // [2][128] normalised, rotated query heads
    bf16* ps = qs + 2 * D;                                                       // [8][32] probabilities of a warp's tile
    bf16* cst = ps + ST_WARPS * 32;                                              // q_norm | k_norm | cos[pos] | sin[pos]
    float* wm = reinterpret_cast<float*>(cst + 4 * D);                           // [8][2]
    float* wl = wm + 16;                                                         // [8][2]
    float* ml = wl + 16;                                                         // [2][2]
    float* ssp = ml + 4;                                                         // [8] partial sums of squares
    unsigned long long* wbest = reinterpret_cast<unsigned long long*>(ssp + 8 + 4);   // [8] (8-byte aligned: 44 floats before it)
    uint64_t* full = reinterpret_cast<uint64_t*>(wbest + ST_WARPS);              // [ST_WARPS][ST_NSLOT]
    int* s_token = reinterpret_cast<int*>(full + ST_WARPS * ST_NSLOT);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int L = a.num_layers;
    const StPlan pl = a.plans[cta];

    if (tid == 0) {
        for (int i = 0; i < ST_WARPS * ST_NSLOT; ++i) mbar_init(&full[i], 1);
        mbar_fence_init();
    }
    __syncthreads();

    uint32_t* xh = reinterpret_cast<uint32_t*>(a.scratch + SC_XH);
    uint32_t* xqkv = reinterpret_cast<uint32_t*>(a.scratch + SC_XQKV);
    uint32_t* xattn = reinterpret_cast<uint32_t*>(a.scratch + SC_XATTN);
    uint32_t* xh1 = reinterpret_cast<uint32_t*>(a.scratch + SC_XH1);
    uint32_t* xact = reinterpret_cast<uint32_t*>(a.scratch + SC_XACT);
    unsigned long long* xpart = reinterpret_cast<unsigned long long*>(a.scratch + SC_XPART);
    unsigned long long* xlm = reinterpret_cast<unsigned long long*>(a.scratch + SC_XLM);
    uint32_t* epoch = reinterpret_cast<uint32_t*>(a.scratch + SC_EPOCH);

    const uint32_t epoch0 = ld_relaxed_u32(epoch);
    const int pos0 = ld_cg_i32(a.pos0);
    // every CTA takes the same decision: nothing is launched half-way
    if (pos0 < 0 || pos0 + a.n_steps > a.max_seq || pos0 + a.n_steps > a.max_split * ST_KV_CAP) {
        if (cta == 0 && tid == 0) atomicOr(a.status, MQ_STATUS_BAD_POSITION);
        return;
    }

    Poller po{a.status, false};
    po.refresh();
    const bool timing = a.dbg != nullptr && tid == 0;
    // this warp's stream and ring; the first ST_NSLOT units are requested at once
    WRing rg;
    {
        size_t woff = 0;
        for (int v = 0; v < warp; ++v) woff += (size_t)st_step_units(pl, v, L) * ST_UNIT;
        rg.base = smem_u32(ring) + (uint32_t)warp * ST_NSLOT * ST_SLOT_BYTES;
        rg.full = full + warp * ST_NSLOT;
        rg.src = a.packed + pl.stream_off + woff;
        rg.status = a.status;
        rg.slot = 0u;
        rg.parity = 0u;
        rg.sub = 0u;
        rg.cur_n = 0u;
        rg.cidx = 0u;
        rg.fidx = 0u;
        rg.step_units = st_step_units(pl, warp, L);
        rg.left = rg.step_units * (uint32_t)a.n_steps;
        for (int k = 0; k < ST_NSLOT && rg.left; ++k) rg.fetch((uint32_t)k, lane);
    }
    unsigned long long* dbg = a.dbg ? a.dbg + (size_t)cta * (L + 1) * ST_STAGES : nullptr;
#define ST_T0() long long t0_ = timing ? clock64() : 0
#define ST_T1(layer, stage)                                                         \
    do {                                                                            \
        if (timing) {                                                               \
            const long long t1_ = clock64();                                        \
            dbg[(size_t)(layer) * ST_STAGES + (stage)] += (unsigned long long)(t1_ - t0_); \
            t0_ = t1_;                                                              \
        }                                                                           \
    } while (0)

    // Tags: phase number p = epoch0 + step * (L + 1) + layer (layer L = the LM head); tag32 = p + 1,
    // tag16 = p % 65535 + 1 (never 0), both advanced incrementally.
    uint32_t t32 = epoch0 + 1u, t16 = epoch0 % 65535u + 1u, t16_prev = 0u;
    auto next_tags = [&]() {
        ++t32;
        t16_prev = t16;
        t16 = t16 == 65535u ? 1u : t16 + 1u;
    };

    const int g = cta % NKV, s_idx = cta / NKV;     // attention item of this CTA
    const int n_od = 8 * pl.od_ng, n_a = 8 * pl.a_ng, n_gu = 8 * pl.gu_np;

    // K/V rows [c0, c0 + n_cached) of layer l -> padded shared-memory rows, 16 bytes per copy
    auto kv_prefetch = [&](int layer, const AttPlan& ap) {
        if (ap.active && ap.n_cached > 0) {
            const size_t head_off = ((size_t)(layer * NKV + g) * a.max_seq + ap.c0) * D;
            const bf16* ksrc = a.k_cache + head_off;
            const bf16* vsrc = a.v_cache + head_off;
            for (int i = tid; i < ap.n_cached * 16; i += ST_THREADS) {
                const int r = i >> 4, c = i & 15;
                cp_async16(kt + (size_t)r * ST_KV_LD + c * 8, ksrc + (size_t)r * D + c * 8);
                cp_async16(vt + (size_t)r * ST_KV_LD + c * 8, vsrc + (size_t)r * D + c * 8);
            }
        }
        cp_async_commit();
    };

    int token = a.forced ? ld_cg_i32(a.forced) : ld_cg_i32(a.first_token);
    kv_prefetch(0, att_plan(cta, pos0, a.max_split));

    for (int step = 0; step < a.n_steps; ++step) {
        const int pos = pos0 + step;
        const AttPlan ap = att_plan(cta, pos, a.max_split);
        if (cta == 0 && tid == 0 && (token < 0 || token >= a.vocab)) atomicOr(a.status, MQ_STATUS_BAD_TOKEN);
        token = min(max(token, 0), a.vocab - 1);
        const bf16* erow = a.embed + (size_t)token * H;
        float resid = 0.f;                               // residual stream of row od_row0 + tid (tid < n_od)
        if (tid < n_od) resid = bf2f(erow[pl.od_row0 + tid]);

        for (int l = 0; l < L; ++l) {
            const bf16* nrm = a.norms + (size_t)l * NORM_STRIDE;
            ST_T0();

            // ---------------- phase A: RMSNorm + rows of [Wq;Wk;Wv]
            if (n_a > 0) {
                uint2 wv = make_uint2(0u, 0u);
                float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
                if (tid < ST_VT) {
                    wv = __ldg(reinterpret_cast<const uint2*>(nrm + 4 * tid));              // input_layernorm
                    if (l == 0) {
                        const uint2 u = __ldg(reinterpret_cast<const uint2*>(erow + 4 * tid));
                        v0 = bf_lo(u.x); v1 = bf_hi(u.x); v2 = bf_lo(u.y); v3 = bf_hi(u.y);
                    } else {
                        const uint4 u = po.words4(xh + 4 * tid, t16_prev);
                        v0 = bf_hi(u.x); v1 = bf_hi(u.y); v2 = bf_hi(u.z); v3 = bf_hi(u.w);
                    }
                    ST_T1(l, 0);
                    const float part = warp_sum(fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, v3 * v3))));
                    if (lane == 0) ssp[warp] = part;
                }
                consumer_bar();
                if (tid < ST_VT) {
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < ST_VW; ++i) ss += ssp[i];
                    const float r = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
                    uint2 o;
                    o.x = pack_bf16x2(rbf(bf_lo(wv.x) * rbf(v0 * r)), rbf(bf_hi(wv.x) * rbf(v1 * r)));
                    o.y = pack_bf16x2(rbf(bf_lo(wv.y) * rbf(v2 * r)), rbf(bf_hi(wv.y) * rbf(v3 * r)));
                    *reinterpret_cast<uint2*>(xs + 4 * tid) = o;
                }
                consumer_bar();
                gemv_phase(rg, pl.a_ng >> 1, pl.a_ng & 1, H, smem_u32(xs), red);
                consumer_bar();
                if (tid < n_a) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) s += red[w * ST_RED_ROWS + tid];
                    publish(xqkv, pl.a_row0 + tid, rbf(s), t16);
                }
                ST_T1(l, 1);
            }

            // ---------------- phase B: attention item (g, split) of this CTA
            if (ap.active) {
                const int n = ap.n;
                const size_t head_off = ((size_t)(l * NKV + g) * a.max_seq) * D;
                // q_norm | k_norm | cos[pos] | sin[pos] do not depend on the hop: fetch them first
                if (tid >= 128 && tid < 192) {
                    const int v = (tid - 128) >> 4, c = tid & 15;
                    const bf16* src = v == 0 ? nrm + 2 * H : v == 1 ? nrm + 2 * H + D
                                    : v == 2 ? a.cos + (size_t)pos * D : a.sin + (size_t)pos * D;
                    *reinterpret_cast<uint4*>(cst + v * D + c * 8) = __ldg(reinterpret_cast<const uint4*>(src + c * 8));
                }
                // raw q(2g), q(2g+1) for every split; k(g), v(g) for the split that owns the new position
                if (tid < 64) {
                    const uint4 v = po.words4(xqkv + 2 * g * D + 4 * tid, t16);
                    *reinterpret_cast<uint2*>(raw + 4 * tid) = tagged_to_bf16x4(v);
                } else if (tid < 128 && ap.is_last) {
                    const int c = tid - 64;                                   // 0..31 k, 32..63 v
                    const int base = c < 32 ? QSZ + g * D + 4 * c : QSZ + KVSZ + g * D + 4 * (c - 32);
                    const uint4 v = po.words4(xqkv + base, t16);
                    *reinterpret_cast<uint2*>(raw + 2 * D + 4 * c) = tagged_to_bf16x4(v);
                }
                ST_T1(l, 2);
                cp_async_wait_all();
                consumer_bar();
                if (warp < 2) {
                    float lo[2], hi[2];
                    norm_rope_smem(raw + warp * D, cst, cst + 2 * D, cst + 3 * D, lane, lo, hi);
                    *reinterpret_cast<uint32_t*>(qs + warp * D + 2 * lane) = pack_bf16x2(lo[0], lo[1]);
                    *reinterpret_cast<uint32_t*>(qs + warp * D + 64 + 2 * lane) = pack_bf16x2(hi[0], hi[1]);
                } else if (warp == 2 && ap.is_last) {
                    float lo[2], hi[2];
                    norm_rope_smem(raw + 2 * D, cst + D, cst + 2 * D, cst + 3 * D, lane, lo, hi);
                    const uint32_t plo = pack_bf16x2(lo[0], lo[1]), phi = pack_bf16x2(hi[0], hi[1]);
                    bf16* krow = kt + (size_t)(n - 1) * ST_KV_LD;
                    *reinterpret_cast<uint32_t*>(krow + 2 * lane) = plo;
                    *reinterpret_cast<uint32_t*>(krow + 64 + 2 * lane) = phi;
                    bf16* gk = a.k_cache + head_off + (size_t)pos * D;
                    *reinterpret_cast<uint32_t*>(gk + 2 * lane) = plo;
                    *reinterpret_cast<uint32_t*>(gk + 64 + 2 * lane) = phi;
                } else if (warp == 3 && ap.is_last) {
                    const uint2 u = *reinterpret_cast<const uint2*>(raw + 3 * D + 4 * lane);
                    *reinterpret_cast<uint2*>(vt + (size_t)(n - 1) * ST_KV_LD + 4 * lane) = u;
                    *reinterpret_cast<uint2*>(a.v_cache + head_off + (size_t)pos * D + 4 * lane) = u;
                } else if (warp >= 4) {
                    // rows between n and the end of the last 16-position tile are multiplied by p = 0
                    const int n16 = (n + 15) & ~15;
                    for (int i = (warp - 4) * 32 + lane; i < (n16 - n) * 16; i += (ST_WARPS - 4) * 32)
                        *reinterpret_cast<uint4*>(vt + (size_t)(n + (i >> 4)) * ST_KV_LD + (i & 15) * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
                consumer_bar();
                // a warp takes 16-position tiles warp, warp + 8, ..: scores = K_tile . q on the tensor
                // cores (positions are the M dimension, the two heads two of the eight N columns),
                // softmax of the tile, probabilities to bf16, out += P . V_tile
                {
                    const int gi = lane >> 2, ti = lane & 3;
                    const float scale = 0.08838834764831845f;  // 1/sqrt(128)
                    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
                    float o[16][4];
#pragma unroll
                    for (int j = 0; j < 16; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
                    const uint32_t qaddr = smem_u32(qs) + (uint32_t)((gi & 1) * D + 2 * ti) * 2u;
                    bf16* pw = ps + warp * 32;
                    for (int tile = warp; tile * 16 < n && warp < ST_VW; tile += ST_VW) {
                        const uint32_t rowoff = (uint32_t)(((tile * 16 + (lane & 15)) * ST_KV_LD + (lane >> 4) * 8) * 2);
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks) {
                            uint32_t af[4];
                            ldsm4(af, smem_u32(kt) + rowoff + ks * 32);
                            uint32_t b0 = lds32(qaddr + ks * 32), b1 = lds32(qaddr + ks * 32 + 16);
                            if (gi >= 2) { b0 = 0u; b1 = 0u; }
                            mma16816(c, af, b0, b1);
                        }
                        const int p_lo = tile * 16 + gi, p_hi = p_lo + 8;
                        const bool own = ti == 0;
                        const float s00 = (own && p_lo < n) ? c[0] * scale : -1e30f, s01 = (own && p_lo < n) ? c[1] * scale : -1e30f;
                        const float s10 = (own && p_hi < n) ? c[2] * scale : -1e30f, s11 = (own && p_hi < n) ? c[3] * scale : -1e30f;
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
                        const float e00 = (own && p_lo < n) ? expf(s00 - m0) : 0.f, e01 = (own && p_lo < n) ? expf(s01 - m1) : 0.f;
                        const float e10 = (own && p_hi < n) ? expf(s10 - m0) : 0.f, e11 = (own && p_hi < n) ? expf(s11 - m1) : 0.f;
                        float u0 = e00 + e10, u1 = e01 + e11;
#pragma unroll
                        for (int off = 4; off < 32; off <<= 1) {
                            u0 += __shfl_xor_sync(0xffffffffu, u0, off);
                            u1 += __shfl_xor_sync(0xffffffffu, u1, off);
                        }
                        l0 = l0 * cr0 + __shfl_sync(0xffffffffu, u0, 0);
                        l1 = l1 * cr1 + __shfl_sync(0xffffffffu, u1, 0);
                        if (own) {
                            pw[gi] = __float2bfloat16_rn(e00); pw[gi + 8] = __float2bfloat16_rn(e10);
                            pw[16 + gi] = __float2bfloat16_rn(e01); pw[16 + gi + 8] = __float2bfloat16_rn(e11);
                        }
                        __syncwarp();
                        uint32_t pa[4] = {0u, 0u, 0u, 0u};      // A = P: row gi is head gi (rows 2..15 are zero)
                        if (gi < 2) {
                            pa[0] = *reinterpret_cast<const uint32_t*>(pw + gi * 16 + 2 * ti);
                            pa[2] = *reinterpret_cast<const uint32_t*>(pw + gi * 16 + 8 + 2 * ti);
                        }
                        const float crg = gi == 0 ? cr0 : cr1;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint32_t bv[4];
                            ldsm4_t(bv, smem_u32(vt) + rowoff + j * 32);
                            o[2 * j][0] *= crg; o[2 * j][1] *= crg; o[2 * j + 1][0] *= crg; o[2 * j + 1][1] *= crg;
                            mma16816(o[2 * j], pa, bv[0], bv[1]);
                            mma16816(o[2 * j + 1], pa, bv[2], bv[3]);
                        }
                        __syncwarp();
                    }
                    if (lane == 0 && warp < ST_VW) { wm[warp * 2] = m0; wm[warp * 2 + 1] = m1; wl[warp * 2] = l0; wl[warp * 2 + 1] = l1; }
                    if (gi < 2 && warp < ST_VW) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            *reinterpret_cast<float2*>(wacc + (warp * 2 + gi) * D + j * 8 + 2 * ti) = make_float2(o[j][0], o[j][1]);
                    }
                }
                consumer_bar();
                const int hh = (tid >> 7) & 1, d = tid & 127;
                const bool vthread = tid < ST_VT;              // the merge, the publishing and the split merge are the vector threads' work
                float acc = 0.f;
                if (vthread) {
                    float M = -1e30f;
#pragma unroll
                    for (int w8 = 0; w8 < ST_VW; ++w8) M = fmaxf(M, wm[w8 * 2 + hh]);
                    float lsum = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < ST_VW; ++w8) {
                        const float f = expf(wm[w8 * 2 + hh] - M);
                        lsum = fmaf(wl[w8 * 2 + hh], f, lsum);
                        acc = fmaf(wacc[(w8 * 2 + hh) * D + d], f, acc);
                    }
                    if (d == 0) { ml[hh * 2] = M; ml[hh * 2 + 1] = lsum; }
                }
                consumer_bar();        // (M, l) published; every read of kt / vt / wacc of this layer is done
                const int qhead = 2 * g + hh;
                if (!vthread) {
                    // warps 8.. have nothing to publish
                } else if (ap.n_act == 1) {
                    publish(xattn, qhead * D + d, rbf(acc / ml[hh * 2 + 1]), t16);
                    ST_T1(l, 3);
                } else {
                    // split-KV: publish the partial; the CTAs of splits 0 and 1 merge head 0 and head 1
                    const size_t pbase = (((size_t)g * ST_MAX_SPLIT + s_idx) * 2 + hh) * ST_PART;
                    publish_u32(xpart, pbase + 2 + d, __float_as_uint(acc), t32);
                    if (d == 0) {
                        publish_u32(xpart, pbase, __float_as_uint(ml[hh * 2]), t32);
                        publish_u32(xpart, pbase + 1, __float_as_uint(ml[hh * 2 + 1]), t32);
                    }
                    ST_T1(l, 3);
                    if (s_idx < 2 && tid < D) {
                        const int mh = s_idx;                             // the head this CTA merges
                        const unsigned long long* hb = xpart + ((size_t)g * ST_MAX_SPLIT * 2 + mh) * ST_PART;
                        constexpr size_t SPLIT_STRIDE = 2 * ST_PART;
                        // (m, l) of split `lane` (n_act <= 18 < 32): one round trip for the warp
                        float mj = -INFINITY, lj = 0.f;
                        if (lane < ap.n_act) {
                            mj = po.f32(hb + (size_t)lane * SPLIT_STRIDE, t32);
                            lj = po.f32(hb + (size_t)lane * SPLIT_STRIDE + 1, t32);
                        }
                        const float M = warp_max(mj);
                        const float fj = (lane < ap.n_act) ? expf(mj - M) : 0.f;
                        const float den = warp_sum(lj * fj);
                        // acc[d] of every split: all loads are issued before the first tag check
                        unsigned long long rawv[ST_MAX_SPLIT];
#pragma unroll
                        for (int j = 0; j < ST_MAX_SPLIT; ++j)
                            if (j < ap.n_act) rawv[j] = ld_relaxed_u64(hb + (size_t)j * SPLIT_STRIDE + 2 + tid);
                        float num = 0.f;
#pragma unroll
                        for (int j = 0; j < ST_MAX_SPLIT; ++j) {
                            const float f = __shfl_sync(0xffffffffu, fj, j);
                            if (j < ap.n_act) {
                                float v = __uint_as_float((uint32_t)rawv[j]);
                                if ((uint32_t)(rawv[j] >> 32) != t32) v = po.f32(hb + (size_t)j * SPLIT_STRIDE + 2 + tid, t32);
                                num = fmaf(v, f, num);
                            }
                        }
                        publish(xattn, (2 * g + mh) * D + tid, rbf(num / den), t16);
                    }
                    ST_T1(l, 4);
                }
                if (ap.is_last) __threadfence();   // the new K/V rows are read by other CTAs in later steps
            }
            // K/V rows of the next attention phase (their positions were written by earlier steps)
            if (l + 1 < L) kv_prefetch(l + 1, ap);
            else if (step + 1 < a.n_steps) kv_prefetch(0, att_plan(cta, pos + 1, a.max_split));

            // ---------------- phase C: rows of Wo + residual
            if (n_od > 0) {
                poll_units<QSZ>(po, xattn, t16, xs, warp, lane);    // the columns of this warp's units
                ST_T1(l, 5);
                gemv_phase(rg, 0, pl.od_ng, QSZ, smem_u32(xs), red);
                consumer_bar();
                if (tid < n_od) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) s += red[w * ST_RED_ROWS + tid];
                    resid = rbf(resid + rbf(s));
                    publish(xh1, pl.od_row0 + tid, resid, t16);
                }
                ST_T1(l, 6);
            }

            // ---------------- phase D: RMSNorm + gate / up rows + SiLU * up
            if (n_gu > 0) {
                uint2 wv = make_uint2(0u, 0u);
                float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
                if (tid < ST_VT) {
                    wv = __ldg(reinterpret_cast<const uint2*>(nrm + H + 4 * tid));          // post_attention_layernorm
                    const uint4 u = po.words4(xh1 + 4 * tid, t16);
                    v0 = bf_hi(u.x); v1 = bf_hi(u.y); v2 = bf_hi(u.z); v3 = bf_hi(u.w);
                    ST_T1(l, 7);
                    const float part = warp_sum(fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, v3 * v3))));
                    if (lane == 0) ssp[warp] = part;
                }
                consumer_bar();
                if (tid < ST_VT) {
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < ST_VW; ++i) ss += ssp[i];
                    const float r = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
                    uint2 o;
                    o.x = pack_bf16x2(rbf(bf_lo(wv.x) * rbf(v0 * r)), rbf(bf_hi(wv.x) * rbf(v1 * r)));
                    o.y = pack_bf16x2(rbf(bf_lo(wv.y) * rbf(v2 * r)), rbf(bf_hi(wv.y) * rbf(v3 * r)));
                    *reinterpret_cast<uint2*>(xs + 4 * tid) = o;
                }
                consumer_bar();
                gemv_phase(rg, pl.gu_np, 0, H, smem_u32(xs), red);
                consumer_bar();
                if (tid < n_gu) {
                    const int t = tid >> 3, i = tid & 7;
                    float gs = 0.f, us = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) {
                        gs += red[w * ST_RED_ROWS + t * 16 + i];
                        us += red[w * ST_RED_ROWS + t * 16 + 8 + i];
                    }
                    const float act = rbf(silu_f32(rbf(gs)));
                    publish(xact, pl.gu_row0 + tid, rbf(act * rbf(us)), t16);
                }
                ST_T1(l, 8);
            }

            // ---------------- phase E: rows of Wd + residual
            if (n_od > 0) {
                poll_units<I>(po, xact, t16, xs, warp, lane);       // the columns of this warp's units
                ST_T1(l, 9);
                gemv_phase(rg, 0, pl.od_ng, I, smem_u32(xs), red);
                consumer_bar();
                if (tid < n_od) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) s += red[w * ST_RED_ROWS + tid];
                    resid = rbf(resid + rbf(s));
                    publish(xh, pl.od_row0 + tid, resid, t16);
                }
                ST_T1(l, 10);
            }
            next_tags();
        }

        // ---------------- final RMSNorm + LM head tiles + arg-max
        {
            ST_T0();
            uint2 wv = make_uint2(0u, 0u);
            float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
            if (tid < ST_VT) {
                wv = __ldg(reinterpret_cast<const uint2*>(a.final_norm + 4 * tid));
                const uint4 u = po.words4(xh + 4 * tid, t16_prev);
                v0 = bf_hi(u.x); v1 = bf_hi(u.y); v2 = bf_hi(u.z); v3 = bf_hi(u.w);
                ST_T1(L, 11);
                const float part = warp_sum(fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, v3 * v3))));
                if (lane == 0) ssp[warp] = part;
            }
            consumer_bar();
            if (tid < ST_VT) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < ST_VW; ++i) ss += ssp[i];
                const float r = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
                uint2 o;
                o.x = pack_bf16x2(rbf(bf_lo(wv.x) * rbf(v0 * r)), rbf(bf_hi(wv.x) * rbf(v1 * r)));
                o.y = pack_bf16x2(rbf(bf_lo(wv.y) * rbf(v2 * r)), rbf(bf_hi(wv.y) * rbf(v3 * r)));
                *reinterpret_cast<uint2*>(xs + 4 * tid) = o;
            }
            consumer_bar();

            float* lg = nullptr;
            if (a.logits && (a.logits_all || step == a.n_steps - 1)) lg = a.logits + (a.logits_all ? (size_t)step * a.vocab : 0);
            // a warp owns whole tiles (tiles warp, warp + 8, .. of the CTA): 16 units of 4 k-steps each
            const uint32_t xl = smem_u32(xs) + (uint32_t)(lane & 3) * 32u;
            unsigned long long best = 0ull;
#pragma unroll 1
            for (int j = warp; j < pl.lm_nt; j += ST_WARPS) {
                float c[4][4];
#pragma unroll
                for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
#pragma unroll 1
                for (int i = 0; i < ST_LM_TILE_UNITS; ++i) full_unit(rg, c, xl + (uint32_t)i * 128u, lane);
                if ((lane & 3) == 0) {
                    const float lo = rbf((c[0][0] + c[1][0]) + (c[2][0] + c[3][0]));
                    const float hi = rbf((c[0][2] + c[1][2]) + (c[2][2] + c[3][2]));
                    const int r0 = pl.lm_row0 + j * 16 + (lane >> 2), r1 = r0 + 8;
                    if (r0 < a.vocab) {
                        if (lg) lg[r0] = lo;
                        const unsigned long long k = argmax_key64(lo, r0);
                        best = k > best ? k : best;
                    }
                    if (r1 < a.vocab) {
                        if (lg) lg[r1] = hi;
                        const unsigned long long k = argmax_key64(hi, r1);
                        best = k > best ? k : best;
                    }
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
                best = other > best ? other : best;
            }
            if (lane == 0) wbest[warp] = best;
            consumer_bar();
            if (tid == 0) {
                unsigned long long k = 0ull;
                for (int i = 0; i < ST_WARPS; ++i) k = wbest[i] > k ? wbest[i] : k;
                publish_u32(xlm, 2 * (size_t)cta, (uint32_t)(k >> 32), t32);
                publish_u32(xlm, 2 * (size_t)cta + 1, (uint32_t)k, t32);
            }
            ST_T1(L, 12);
            // every CTA reduces the keys of all CTAs itself: no extra hop for the token
            unsigned long long k = 0ull;
            if (tid < grid) {
                const uint32_t hi = __float_as_uint(po.f32(xlm + 2 * (size_t)tid, t32));
                const uint32_t lo = __float_as_uint(po.f32(xlm + 2 * (size_t)tid + 1, t32));
                k = ((unsigned long long)hi << 32) | lo;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, off);
                k = other > k ? other : k;
            }
            consumer_bar();                    // wbest of this step has been read by thread 0
            if (lane == 0) wbest[warp] = k;
            consumer_bar();
            if (tid == 0) {
                unsigned long long kk = 0ull;
                for (int i = 0; i < ST_WARPS; ++i) kk = wbest[i] > kk ? wbest[i] : kk;
                const int next = (int)(0xffffffffu - (uint32_t)(kk & 0xffffffffull));
                *s_token = next;
                if (cta == 0) a.tokens_out[step] = next;
            }
            consumer_bar();
            token = *s_token;
            if (a.forced && step + 1 < a.n_steps) token = ld_cg_i32(a.forced + step + 1);
            ST_T1(L, 13);
        }
        next_tags();
    }
    if (cta == 0 && tid == 0) st_relaxed_u32(epoch, epoch0 + (uint32_t)(a.n_steps * (L + 1)));
    // a kernel that is draining after an expired wait may still have bulk copies on their way to
    // this CTA's shared memory: give them time to land before the memory is handed back
    if (ld_relaxed_u32(a.status) & MQ_STATUS_WAIT_TIMEOUT)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
#undef ST_T0
#undef ST_T1
}

// ------------------------------------------------------------------ weight packing
// Every 32-bit word of a warp's stream is two adjacent bf16 of one weight row, placed where the
// mma A fragment of its block expects them (layout: see gemv_phase).
__device__ __forceinline__ uint32_t pack_word(const bf16* W, int ld, int row, int col) {
    return *reinterpret_cast<const uint32_t*>(W + (size_t)row * ld + col);
}

// (row within the tile, column) of word `wd` (0..511) of a unit; warp_col0 = first column of the warp
__device__ __forceinline__ void unit_word_pos(bool full_tile, int unit_in_tile, int warp_col0, uint32_t wd, int& trow, int& col) {
    const int blk = (int)(wd >> 7), ln = (int)((wd & 127u) >> 2), reg = (int)(wd & 3u);
    const int g = ln >> 2, tig = ln & 3;
    if (full_tile) {
        trow = g + ((reg & 1) ? 8 : 0);
        col = warp_col0 + 64 * unit_in_tile + 16 * tig + 4 * blk + ((reg & 2) ? 2 : 0);
    } else {
        trow = g;
        col = warp_col0 + 128 * unit_in_tile + 32 * tig + 8 * blk + 2 * reg;
    }
}

// grid (CTAs, warps, z); one layer of one warp's stream per (x, y)
__global__ void k_pack_layer(const StPlan* plans, MqLayerWeights w, uint8_t* packed, int layer, int num_layers) {
    const StPlan pl = plans[blockIdx.x];
    const int warp = blockIdx.y;
    size_t woff = 0;
    for (int v = 0; v < warp; ++v) woff += (size_t)st_step_units(pl, v, num_layers) * ST_UNIT;
    const uint32_t layer_units = st_layer_units(pl, warp);
    uint32_t* dst = reinterpret_cast<uint32_t*>(packed + pl.stream_off + woff + (size_t)layer * layer_units * ST_UNIT);
    const uint32_t nwords = layer_units * (ST_UNIT / 4);
    // units of the four phases, in stream order
    const int ng[4] = {pl.a_ng, pl.od_ng, 2 * pl.gu_np, pl.od_ng};
    const int Ks[4] = {H, QSZ, H, I};
    for (uint32_t wi = blockIdx.z * blockDim.x + threadIdx.x; wi < nwords; wi += gridDim.z * blockDim.x) {
        uint32_t unit = wi / (ST_UNIT / 4);
        const uint32_t wd = wi % (ST_UNIT / 4);
        int phase = 0;
        while (phase < 3 && unit >= st_phase_units(Ks[phase], ng[phase], warp)) { unit -= st_phase_units(Ks[phase], ng[phase], warp); ++phase; }
        const int K = Ks[phase];
        const int ntf = ng[phase] >> 1;
        const uint32_t upt = (uint32_t)(K / (64 * ST_WARPS));    // units of this warp per full tile
        const bool full_tile = unit < (uint32_t)ntf * upt;
        const int tile = full_tile ? (int)(unit / upt) : ntf;
        int trow, col;
        if (full_tile) unit_word_pos(true, (int)(unit % upt), warp * (K / ST_WARPS), wd, trow, col);
        else unit_word_pos(false, 0, (warp + (int)(unit - (uint32_t)ntf * upt) * ST_WARPS) * 128, wd, trow, col);   // half-tile unit warp + k W
        const bf16* W;
        int row;
        if (phase == 0) {
            const int r = pl.a_row0 + tile * 16 + trow;
            if (r < QSZ) { W = (const bf16*)w.q_proj; row = r; }
            else if (r < QSZ + KVSZ) { W = (const bf16*)w.k_proj; row = r - QSZ; }
            else { W = (const bf16*)w.v_proj; row = r - QSZ - KVSZ; }
        } else if (phase == 2) {
            W = trow < 8 ? (const bf16*)w.gate_proj : (const bf16*)w.up_proj;
            row = pl.gu_row0 + tile * 8 + (trow & 7);
        } else {
            W = phase == 1 ? (const bf16*)w.o_proj : (const bf16*)w.down_proj;
            row = pl.od_row0 + tile * 16 + trow;
        }
        dst[wi] = pack_word(W, K, row, col);
    }
}

__global__ void k_pack_lm(const StPlan* plans, const bf16* lm_head, uint8_t* packed, int num_layers, int vocab) {
    const StPlan pl = plans[blockIdx.x];
    const int warp = blockIdx.y;
    size_t woff = 0;
    for (int v = 0; v < warp; ++v) woff += (size_t)st_step_units(pl, v, num_layers) * ST_UNIT;
    uint32_t* dst = reinterpret_cast<uint32_t*>(packed + pl.stream_off + woff + (size_t)num_layers * st_layer_units(pl, warp) * ST_UNIT);
    const uint32_t nwords = st_lm_tiles(pl, warp) * ST_LM_TILE_UNITS * (ST_UNIT / 4);
    for (uint32_t wi = blockIdx.z * blockDim.x + threadIdx.x; wi < nwords; wi += gridDim.z * blockDim.x) {
        const uint32_t unit = wi / (ST_UNIT / 4), wd = wi % (ST_UNIT / 4);
        const int k = (int)(unit / ST_LM_TILE_UNITS), uit = (int)(unit % ST_LM_TILE_UNITS);
        int trow, col;
        unit_word_pos(true, uit, 0, wd, trow, col);
        const int row = pl.lm_row0 + (warp + ST_WARPS * k) * 16 + trow;
        dst[wi] = row < vocab ? pack_word(lm_head, H, row, col) : 0u;
    }
}

__global__ void k_pack_norms(MqLayerWeights w, bf16* dst) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < H) { dst[i] = ((const bf16*)w.input_layernorm)[i]; dst[H + i] = ((const bf16*)w.post_attn_layernorm)[i]; }
    if (i < D) { dst[2 * H + i] = ((const bf16*)w.q_norm)[i]; dst[2 * H + D + i] = ((const bf16*)w.k_norm)[i]; }
}

// ------------------------------------------------------------------ host side
static size_t st_smem_bytes() {
    return (size_t)ST_WARPS * ST_NSLOT * ST_SLOT_BYTES + (size_t)2 * ST_KV_CAP * ST_KV_LD * 2 + (size_t)I * 2 + (size_t)ST_WARPS * ST_RED_ROWS * 4 +
           (4 * D + 2 * D + ST_WARPS * 32 + 4 * D) * 2 + (16 + 16 + 4 + 8 + 4) * 4 + ST_WARPS * 8 + ST_WARPS * ST_NSLOT * 8 + 16;
}

constexpr size_t ST_HDR_PLANS = 0;
static size_t st_hdr_norms() { return ((size_t)ST_MAX_GRID * sizeof(StPlan) + 255) & ~(size_t)255; }
static size_t st_hdr_bytes(int num_layers) {
    return (st_hdr_norms() + (size_t)num_layers * NORM_STRIDE * 2 + 4095) / 4096 * 4096;
}

// Deals the rows out.  A step is bound by its chain of dependent phases, not by a CTA's total
// bytes: every phase lasts as long as its most loaded CTA, so each phase is spread as evenly
// as its granularity allows (8-row groups of q|k|v, 8 + 8-row gate/up pairs, 8-row groups of
// Wo / Wd): 3-4 + 1 + 2-3 + 1 on 148 SMs.  CTAs 0..127 own one Wo/Wd group each (the same
// rows in both, so that the residual of those rows stays in a register); the CTAs without one
// take the larger shares of the other two phases.
static int st_make_plans(int grid, int num_layers, int vocab, std::vector<StPlan>& plans, size_t* total_bytes) {
    if (grid < ST_MIN_GRID || grid > ST_MAX_GRID) return MQ_ERR_UNSUPPORTED;
    const int n_od = H / 8, n_a = QKV / 8, n_gu = I / 8;
    plans.assign(grid, StPlan{});
    std::vector<int> pairs(grid, 0), od(grid, 0), ag(grid, 0);
    for (int c = 0; c < grid; ++c) od[c] = c < n_od ? 1 : 0;
    // the larger shares go to the highest-numbered CTAs first (those without Wo / Wd rows)
    for (int c = 0; c < grid; ++c) {
        pairs[c] = n_gu / grid + (grid - 1 - c < n_gu % grid ? 1 : 0);
        ag[c] = n_a / grid;
    }
    // q|k|v extras: prefer CTAs that did not get an extra gate/up pair, from the top down
    int extra = n_a % grid;
    for (int pass = 0; pass < 2 && extra > 0; ++pass)
        for (int c = grid - 1; c >= 0 && extra > 0; --c) {
            const bool has_extra_pair = pairs[c] > n_gu / grid;
            if (ag[c] == n_a / grid && (pass == 1 || !has_extra_pair || od[c] == 0)) { ag[c] += 1; --extra; }
        }
    for (int c = 0; c < grid; ++c)
        if (pairs[c] > ST_MAX_TILES) return MQ_ERR_UNSUPPORTED;
    const int lm_tiles = (vocab + 15) / 16;
    int a_next = 0, od_next = 0, gu_next = 0, lm_next = 0;
    size_t off = st_hdr_bytes(num_layers);
    for (int c = 0; c < grid; ++c) {
        StPlan& p = plans[c];
        p.a_row0 = 8 * a_next; p.a_ng = ag[c]; a_next += ag[c];
        p.od_row0 = 8 * od_next; p.od_ng = od[c]; od_next += od[c];
        p.gu_row0 = 8 * gu_next; p.gu_np = pairs[c]; gu_next += pairs[c];
        p.lm_nt = lm_tiles / grid + (c < lm_tiles % grid ? 1 : 0);
        p.lm_row0 = 16 * lm_next; lm_next += p.lm_nt;
        if (p.a_ng > 2 * ST_MAX_TILES || p.od_ng > 1) return MQ_ERR_UNSUPPORTED;   // Wo / Wd rows: one 8-row group per CTA at most
        p.layer_units = 0;
        p.stream_off = off;
        for (int wv = 0; wv < ST_WARPS; ++wv) off += (size_t)st_step_units(p, wv, num_layers) * ST_UNIT;
    }
    if (a_next != n_a || od_next != n_od || gu_next != n_gu || lm_next != lm_tiles) return MQ_ERR_UNSUPPORTED;
    *total_bytes = off;
    return MQ_OK;
}

struct StDevice {
    bool ready = false;
    int sm_count = 0;
};
static StDevice g_st_dev[64];

static int st_ensure_device(StDevice** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
    StDevice& st = g_st_dev[dev];
    if (!st.ready) {
        cudaDeviceProp p;
        e = cudaGetDeviceProperties(&p, dev);
        if (e != cudaSuccess) return (int)e;
        if (p.major != 10 || p.multiProcessorCount < ST_MIN_GRID || p.multiProcessorCount > ST_MAX_GRID || !p.cooperativeLaunch)
            return MQ_ERR_UNSUPPORTED;
        st.sm_count = p.multiProcessorCount;
        e = cudaFuncSetAttribute(k_decode_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem_bytes());
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_stream, ST_THREADS, st_smem_bytes());
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return MQ_ERR_UNSUPPORTED;
        st.ready = true;
    }
    *out = &st;
    return MQ_OK;
}

}  // namespace mq

using namespace mq;


extern "C" size_t mq_stream_scratch_bytes(void) { return SC_BYTES; }

extern "C" int mq_stream_max_context(void) {
    StDevice* st = nullptr;
    if (st_ensure_device(&st) != MQ_OK) return 0;
    const int ms = st->sm_count / NKV < ST_MAX_SPLIT ? st->sm_count / NKV : ST_MAX_SPLIT;
    return ms * ST_KV_CAP;
}

extern "C" int mq_stream_stage_count(void) { return ST_STAGES; }

extern "C" int mq_stream_grid(void) {
    StDevice* st = nullptr;
    if (st_ensure_device(&st) != MQ_OK) return 0;
    return st->sm_count;
}

extern "C" size_t mq_stream_packed_bytes(const MqModel* model) {
    if (!model || model->num_layers <= 0 || model->vocab_size <= 0) return 0;
    StDevice* st = nullptr;
    if (st_ensure_device(&st) != MQ_OK) return 0;
    std::vector<StPlan> plans;
    size_t total = 0;
    if (st_make_plans(st->sm_count, model->num_layers, model->vocab_size, plans, &total) != MQ_OK) return 0;
    return total;
}

extern "C" int mq_stream_pack(const MqModel* model, void* packed, size_t packed_bytes, void* stream_v) {
    if (!model || !packed || !model->layers || !model->lm_head) return MQ_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(packed) & 255u) != 0) return MQ_ERR_ALIGNMENT;
    StDevice* st = nullptr;
    int rc = st_ensure_device(&st);
    if (rc != MQ_OK) return rc;
    std::vector<StPlan> plans;
    size_t total = 0;
    rc = st_make_plans(st->sm_count, model->num_layers, model->vocab_size, plans, &total);
    if (rc != MQ_OK) return rc;
    if (packed_bytes < total) return MQ_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_v;
    uint8_t* base = static_cast<uint8_t*>(packed);
    cudaError_t e = cudaMemcpyAsync(base + ST_HDR_PLANS, plans.data(), plans.size() * sizeof(StPlan), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(stream);      // `plans` is a host temporary
    if (e != cudaSuccess) return (int)e;
    const StPlan* dplans = reinterpret_cast<const StPlan*>(base + ST_HDR_PLANS);
    bf16* norms = reinterpret_cast<bf16*>(base + st_hdr_norms());
    for (int l = 0; l < model->num_layers; ++l) {
        k_pack_norms<<<(H + 255) / 256, 256, 0, stream>>>(model->layers[l], norms + (size_t)l * NORM_STRIDE);
        k_pack_layer<<<dim3(st->sm_count, ST_WARPS, 2), 256, 0, stream>>>(dplans, model->layers[l], base, l, model->num_layers);
    }
    k_pack_lm<<<dim3(st->sm_count, ST_WARPS, 8), 256, 0, stream>>>(dplans, (const bf16*)model->lm_head, base, model->num_layers, model->vocab_size);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_decode_stream(const MqModel* model, const void* packed, void* k_cache, void* v_cache, void* scratch,
                                       unsigned int* status, const int* first_token, const int* position0,
                                       const int* forced_tokens, int* tokens_out, int n_steps, float* logits, int logits_all,
                                       unsigned long long* stage_cycles, void* stream_v) {
    if (!model || !packed || !k_cache || !v_cache || !scratch || !status || !position0 || !tokens_out) return MQ_ERR_BAD_ARG;
    if (!first_token && !forced_tokens) return MQ_ERR_BAD_ARG;
    if (!model->embed || !model->final_norm || !model->cos_table || !model->sin_table) return MQ_ERR_BAD_ARG;
    if (model->num_layers <= 0 || model->vocab_size <= 0 || model->max_seq_len <= 0 || n_steps <= 0) return MQ_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(packed) & 255u) || (reinterpret_cast<uintptr_t>(scratch) & 255u) ||
        (reinterpret_cast<uintptr_t>(k_cache) & 15u) || (reinterpret_cast<uintptr_t>(v_cache) & 15u))
        return MQ_ERR_ALIGNMENT;
    StDevice* st = nullptr;
    int rc = st_ensure_device(&st);
    if (rc != MQ_OK) return rc;
    const uint8_t* base = static_cast<const uint8_t*>(packed);
    StreamArgs a;
    a.packed = base;
    a.plans = reinterpret_cast<const StPlan*>(base + ST_HDR_PLANS);
    a.norms = reinterpret_cast<const bf16*>(base + st_hdr_norms());
    a.embed = (const bf16*)model->embed;
    a.final_norm = (const bf16*)model->final_norm;
    a.cos = (const bf16*)model->cos_table;
    a.sin = (const bf16*)model->sin_table;
    a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache;
    a.scratch = static_cast<uint8_t*>(scratch);
    a.status = status;
    a.first_token = first_token;
    a.pos0 = position0;
    a.forced = forced_tokens;
    a.tokens_out = tokens_out;
    a.logits = logits;
    a.dbg = stage_cycles;
    a.num_layers = model->num_layers;
    a.vocab = model->vocab_size;
    a.max_seq = model->max_seq_len;
    a.n_steps = n_steps;
    a.logits_all = logits_all;
    a.max_split = st->sm_count / NKV < ST_MAX_SPLIT ? st->sm_count / NKV : ST_MAX_SPLIT;
    void* params[] = {&a};
    return (int)cudaLaunchCooperativeKernel((const void*)k_decode_stream, dim3(st->sm_count), dim3(ST_THREADS), params,
                                            st_smem_bytes(), (cudaStream_t)stream_v);
}
