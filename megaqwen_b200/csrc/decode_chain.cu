// Persistent batch-1 decode chain for sm_100a: ONE cooperative launch runs
// n_steps greedy decode steps (all layers, LM head, arg-max, next embedding).
//
// Why.  A decode step is ~140 dependent phases of ~1.2 us of HBM time each.
// With one kernel per phase (csrc/decode.cu) every hand-over costs a grid
// completion plus a dependent-launch wake-up (~4 us per phase measured).  Here
// the 148 CTAs (one per SM, co-resident by cooperative launch) stay alive and
// exchange activations through small global buffers whose 32-bit words carry
// the bf16 value in the high half and a 16-bit phase tag in the low half: a
// consumer simply re-reads the words it needs until all tags match, so one L2
// round trip transfers data and readiness together and no fence, flag or
// grid-wide barrier exists.  (The reference uses 225 cooperative grid.sync()
// calls per token, csrc/megakernel/fused_decode_ldg_kernel.inl:43-137.)
//
// Weights never depend on activations, so a dedicated producer thread per CTA
// streams that CTA's slices of every phase, in consumption order, through a
// 208 KB shared-memory byte ring with 1-D TMA bulk copies (non-multicast) and
// runs ahead of the consumers by up to the ring size (about one layer), KV-cache
// chunks and LM-head rows included.  HBM traffic therefore continues while the
// consumer warps wait for activations.
//
// Every wait (mbarrier or tag poll) is bounded; on expiry the sticky status
// word is set, all later waits give up at once and the kernel drains.
//
// Arithmetic and rounding points are identical to csrc/decode.cu.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mq_device.cuh"

namespace mq {

constexpr int CH_CONSUMER_WARPS = 8;                      // 8 + 1 producer warp: no SM sub-partition holds more than 3 warps,
                                                          // so threads may use well over 128 registers
constexpr int CH_CONSUMERS = CH_CONSUMER_WARPS * 32;      // 256 threads
constexpr int CH_THREADS = CH_CONSUMERS + 32;             // + producer warp
constexpr int CH_RING_BYTES = 200 * 1024;
constexpr int CH_MAX_LAYERS = 48;                         // layer table copy in shared memory
constexpr int CH_NB = 32;                                 // ring segments in flight (mbarrier pairs)
#ifndef MQ_PR_QKV
#define MQ_PR_QKV 7
#endif
constexpr int PR_QKV = MQ_PR_QKV;                                 // rows per ring piece: 14 KB
#ifndef MQ_PR_O
#define MQ_PR_O 4
#endif
constexpr int PR_O = MQ_PR_O;                                   // 16 KB
#ifndef MQ_PR_GU
#define MQ_PR_GU 4
#endif
constexpr int PR_GU = MQ_PR_GU;                                  // 4 gate + 4 up rows: 16 KB
#ifndef MQ_PR_D
#define MQ_PR_D 2
#endif
constexpr int PR_D = MQ_PR_D;                                   // 12 KB
#ifndef MQ_PR_KV
#define MQ_PR_KV 64
#endif
constexpr int PR_KV = MQ_PR_KV;                                 // cache positions per piece: 16 KB
#ifndef MQ_CH_MAXP
#define MQ_CH_MAXP 6
#endif
constexpr int CH_MAXP = MQ_CH_MAXP;                                // pieces per phase
constexpr int CH_LM_ROWS = 2 * CH_CONSUMER_WARPS;         // LM-head rows per ring segment (32 KB)
constexpr int CH_MIN_GRID = 128;
constexpr int CH_MAX_SPLIT = 16;                          // 8 kv heads x 16 splits = 128 <= grid
constexpr int CH_MAX_CAP = 192;                           // positions per attention CTA
constexpr int CH_MIN_CHUNK = 64;
constexpr int CH_PART = D + 2;
constexpr int CH_REP = 1;                                 // replicas of every exchanged vector (readers per line / 16)
constexpr int CH_XWORDS = H + QKV + QSZ + H + I;          // tagged words per replica

struct ChainArgs {
    const bf16* embed;
    const bf16* final_norm;
    const bf16* lm_head;
    const bf16* cos;
    const bf16* sin;
    const MqLayerWeights* layers;   // device array
    bf16* k_cache;
    bf16* v_cache;
    uint32_t* xh;                   // tagged words [1024]
    uint32_t* xqkv;                 // [4096]
    uint32_t* xattn;                // [2048]
    uint32_t* xh1;                  // [1024]
    uint32_t* xact;                 // [3072]
    unsigned long long* xpart;      // [16 * nsplit * 130] (tag32 << 32 | fp32 bits)
    unsigned long long* xlm;        // [grid * 2]
    uint32_t* epoch;                // [1] persistent phase counter
    unsigned int* status;
    const int* first_token;
    const int* pos0;
    int* tokens_out;                // [n_steps]
    float* logits;                  // optional fp32 [vocab] of the LAST step
    unsigned long long* dbg;        // optional [grid][8] cycle counters (CTA-level stage times)
    int l2_ahead;                   // prefetch the next layer's slices into L2
    int exp_flags;                  // experiments: 1 skip dot products, 2 do not wait for tags
    int num_layers;
    int vocab;
    int max_seq;
    int n_steps;
    int nsplit;
    int chunk_cap;
};

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
// value must already be exactly representable in bf16
// Every value is stored into all CH_REP replicas of the exchange buffers (CTA c reads
// replica c % CH_REP).  Measured on B200: 16 replicas did not shorten the polls and the
// extra stores cost more than they saved, so one replica is used.
__device__ __forceinline__ void publish(uint32_t* dst, int idx, float v, uint32_t tag16) {
    const uint32_t wv = (__float_as_uint(v) & 0xffff0000u) | tag16;
#pragma unroll
    for (int r = 0; r < CH_REP; ++r) st_relaxed_u32(dst + (size_t)r * CH_XWORDS + idx, wv);
}
__device__ __forceinline__ void publish_f32(unsigned long long* dst, size_t idx, float v, uint32_t tag32) {
    st_relaxed_u64(dst + idx, ((unsigned long long)tag32 << 32) | (unsigned long long)__float_as_uint(v));
}

constexpr long long POLL_LIMIT_CYCLES = 400000000LL;

struct Poller {
    unsigned int* status;
    bool aborted;
    bool nowait;
    __device__ __forceinline__ void refresh() { aborted = (ld_relaxed_u32(status) & MQ_STATUS_WAIT_TIMEOUT) != 0; }
    __device__ __forceinline__ void expire() {
        atomicOr(status, MQ_STATUS_WAIT_TIMEOUT);
        aborted = true;
    }
    // 4 consecutive tagged words; returns when all carry `tag16` (or on abort)
    __device__ __forceinline__ uint4 words4(const uint32_t* p, uint32_t tag16) {
        uint4 v = ld_relaxed_v4(p);
        auto ok = [&](const uint4& u) {
            return ((u.x & 0xffffu) == tag16) & ((u.y & 0xffffu) == tag16) & ((u.z & 0xffffu) == tag16) & ((u.w & 0xffffu) == tag16);
        };
        if (ok(v) || aborted || nowait) return v;
        const long long t0 = clock64();
        int it = 0;
        for (;;) {
            v = ld_relaxed_v4(p);
            if (ok(v)) return v;
            if ((++it & 63) == 0) {
                refresh();
                if (aborted) return v;
                if (clock64() - t0 > POLL_LIMIT_CYCLES) { expire(); return v; }
            }
        }
    }
    __device__ __forceinline__ float f32(const unsigned long long* p, uint32_t tag32) {
        unsigned long long v = ld_relaxed_u64(p);
        if ((uint32_t)(v >> 32) == tag32 || aborted || nowait) return __uint_as_float((uint32_t)v);
        const long long t0 = clock64();
        int it = 0;
        for (;;) {
            v = ld_relaxed_u64(p);
            if ((uint32_t)(v >> 32) == tag32) break;
            if ((++it & 63) == 0) {
                refresh();
                if (aborted) break;
                if (clock64() - t0 > POLL_LIMIT_CYCLES) { expire(); break; }
            }
        }
        return __uint_as_float((uint32_t)v);
    }
};

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(CH_CONSUMERS) : "memory"); }

// Gather a tagged vector of `nwords` (multiple of 4) into shared memory as bf16.
__device__ __forceinline__ void poll_vector(Poller& po, const uint32_t* src, int nwords, uint32_t tag16, bf16* dst, int ctid) {
    // up to three 16-byte chunks per thread (3072 words / 256 threads): all loads are
    // issued before the first tag check, stale chunks are then re-polled one by one
    const int nch = nwords / 4;
    uint4 v[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int c = ctid + k * CH_CONSUMERS;
        if (c < nch) v[k] = ld_relaxed_v4(src + 4 * c);
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int c = ctid + k * CH_CONSUMERS;
        if (c < nch) {
            const bool ok = ((v[k].x & 0xffffu) == tag16) & ((v[k].y & 0xffffu) == tag16) & ((v[k].z & 0xffffu) == tag16) & ((v[k].w & 0xffffu) == tag16);
            if (!ok) v[k] = po.words4(src + 4 * c, tag16);
            uint2 o;
            o.x = (v[k].x >> 16) | (v[k].y & 0xffff0000u);
            o.y = (v[k].z >> 16) | (v[k].w & 0xffff0000u);
            *reinterpret_cast<uint2*>(dst + 4 * c) = o;
        }
    }
}

// NR rows at once: independent accumulators and interleaved shuffle reductions,
// so the latency chains of the rows overlap.  Rows with ok[r] == false are skipped.
template <int NR, int NJ>
__device__ __forceinline__ void dots_multi(const bf16* const (&rows)[NR], const bool (&ok)[NR], const float (&x)[NJ * 8], int lane,
                                           float (&out)[NR]) {
    float a0[NR], a1[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) { a0[r] = 0.f; a1[r] = 0.f; }
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            if (ok[r]) {
                const uint4 u = reinterpret_cast<const uint4*>(rows[r])[j * 32 + lane];
                a0[r] = fmaf(bf_lo(u.x), x[j * 8 + 0], a0[r]); a1[r] = fmaf(bf_hi(u.x), x[j * 8 + 1], a1[r]);
                a0[r] = fmaf(bf_lo(u.y), x[j * 8 + 2], a0[r]); a1[r] = fmaf(bf_hi(u.y), x[j * 8 + 3], a1[r]);
                a0[r] = fmaf(bf_lo(u.z), x[j * 8 + 4], a0[r]); a1[r] = fmaf(bf_hi(u.z), x[j * 8 + 5], a1[r]);
                a0[r] = fmaf(bf_lo(u.w), x[j * 8 + 6], a0[r]); a1[r] = fmaf(bf_hi(u.w), x[j * 8 + 7], a1[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = a0[r] + a1[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int r = 0; r < NR; ++r) out[r] += __shfl_xor_sync(0xffffffffu, out[r], o);
    }
}

// Cooperative RMSNorm of a 1024-wide vector: threads 0..255 hold 4 elements each
// (v, valid when has), the sum of squares is reduced through `red`, each thread
// normalises its own elements with the weight vector `wn` (shared memory) and
// stores bf16 results to `dst`.  Two consumer barriers; every element is
// normalised exactly once per CTA.
__device__ __forceinline__ void coop_rmsnorm_store(const float (&v)[4], bool has, const bf16* wn, bf16* dst, float* red,
                                                   int ctid, int lane, int warp) {
    float ss = has ? (v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]) : 0.f;
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    consumer_bar();
    if (has) {
        float tot = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) tot += red[w8];
        const float r = 1.0f / sqrtf(tot * (1.0f / H) + RMS_EPS);
        const uint2 wu = *reinterpret_cast<const uint2*>(wn + 4 * ctid);
        uint2 o;
        o.x = pack_bf16x2(rbf(bf_lo(wu.x) * rbf(v[0] * r)), rbf(bf_hi(wu.x) * rbf(v[1] * r)));
        o.y = pack_bf16x2(rbf(bf_lo(wu.y) * rbf(v[2] * r)), rbf(bf_hi(wu.y) * rbf(v[3] * r)));
        *reinterpret_cast<uint2*>(dst + 4 * ctid) = o;
    }
    consumer_bar();
}

// lane slice of an NJ*256-wide bf16 vector in shared memory -> fp32 registers
template <int NJ>
__device__ __forceinline__ void load_x_smem(float (&x)[NJ * 8], const bf16* src, int lane) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const uint4 u = *reinterpret_cast<const uint4*>(src + j * 256 + lane * 8);
        x[j * 8 + 0] = bf_lo(u.x); x[j * 8 + 1] = bf_hi(u.x);
        x[j * 8 + 2] = bf_lo(u.y); x[j * 8 + 3] = bf_hi(u.y);
        x[j * 8 + 4] = bf_lo(u.z); x[j * 8 + 5] = bf_hi(u.z);
        x[j * 8 + 6] = bf_lo(u.w); x[j * 8 + 7] = bf_hi(u.w);
    }
}
__device__ __forceinline__ void load_x_global_ro(float (&x)[32], const bf16* src, int lane) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(src + j * 256 + lane * 8));
        x[j * 8 + 0] = bf_lo(u.x); x[j * 8 + 1] = bf_hi(u.x);
        x[j * 8 + 2] = bf_lo(u.y); x[j * 8 + 3] = bf_hi(u.y);
        x[j * 8 + 4] = bf_lo(u.z); x[j * 8 + 5] = bf_hi(u.z);
        x[j * 8 + 6] = bf_lo(u.w); x[j * 8 + 7] = bf_hi(u.w);
    }
}

// per-head RMSNorm + RoPE on a raw head held in shared memory (bf16[128])
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
        lo[e] = rbf(rbf(nl * clo[e]) + rbf(-nh * slo[e]));
        hi[e] = rbf(rbf(nh * chi[e]) + rbf(nl * shi[e]));
    }
}

// ------------------------------------------------------------------ ring bookkeeping
// Producer and consumers walk the same static list of segments and compute the
// same offsets: a segment is placed at `head`, or at 0 if it would cross the end.
struct RingCursor {
    uint32_t seg;    // running segment index
    uint32_t head;   // next free byte
    __device__ __forceinline__ uint32_t place(uint32_t bytes) {
        uint32_t off = head;
        if (off + bytes > (uint32_t)CH_RING_BYTES) off = 0;
        head = off + bytes;
        ++seg;
        return off;
    }
};

// A phase's slice is cut into pieces of `pr` rows so that ring space is used
// densely; all pieces of a phase are placed up front.
struct Pieces {
    uint32_t off[CH_MAXP];
    uint32_t k0;
    int np;
};
__device__ __forceinline__ Pieces place_pieces(RingCursor& rc, int rows, int pr, uint32_t row_bytes) {
    Pieces P;
    P.k0 = rc.seg;
    P.np = (rows + pr - 1) / pr;
#pragma unroll
    for (int p = 0; p < CH_MAXP; ++p)
        if (p < P.np) P.off[p] = rc.place((uint32_t)min(pr, rows - p * pr) * row_bytes);
    return P;
}
__device__ __forceinline__ uint32_t piece_off(const Pieces& P, int p) {
    uint32_t o = P.off[0];
#pragma unroll
    for (int j = 1; j < CH_MAXP; ++j) o = (p == j) ? P.off[j] : o;
    return o;
}

struct Geometry {
    int q0, qn;    // rows of [Wq;Wk;Wv]
    int o0, on;    // rows of Wo and Wd
    int g0, gn;    // rows of Wg / Wu
    int v0, vn;    // rows of the LM head
    int att_g, att_s;  // attention item, att_g < 0 if this CTA never runs attention
};

__device__ __forceinline__ void split_rows(int total, int cta, int grid, int& r0, int& n) {
    r0 = (int)(((long long)cta * total) / grid);
    n = (int)(((long long)(cta + 1) * total) / grid) - r0;
}

struct AttPlan {
    int n_act, chunk, c0, n, n_cached;
    bool active, is_last;
};
__device__ __forceinline__ AttPlan att_plan(const Geometry& ge, int pos, int nsplit, bool skip = false) {
    AttPlan p;
    const int len = pos + 1;
    int chunk = (len + nsplit - 1) / nsplit;
    p.chunk = max(CH_MIN_CHUNK, (chunk + 15) & ~15);
    p.n_act = (len + p.chunk - 1) / p.chunk;
    p.active = ge.att_g >= 0 && ge.att_s < p.n_act && !skip;
    p.c0 = ge.att_s * p.chunk;
    p.n = p.active ? min(len, p.c0 + p.chunk) - p.c0 : 0;
    p.is_last = p.active && ge.att_s == p.n_act - 1;
    p.n_cached = p.is_last ? p.n - 1 : p.n;
    return p;
}

// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(CH_THREADS, 1) k_decode_chain(ChainArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* ring = smem_raw;
    bf16* xbuf = reinterpret_cast<bf16*>(smem_raw + CH_RING_BYTES);          // [2][3072]
    float* sc = reinterpret_cast<float*>(xbuf + 2 * I);                       // [2][CH_MAX_CAP]
    float* qh = sc + 2 * CH_MAX_CAP;                                          // [2][128]
    float* accb = qh + 2 * D;                                                 // [6][128]
    float* ml = accb + 6 * D;                                                 // [4]
    float* part = ml + 4;                                                     // [8][4]
    float* red = part + 32;                                                   // [16] warp partial sums
    unsigned long long* wbest = reinterpret_cast<unsigned long long*>(red + 16);   // [12] (8-byte aligned)
    uint64_t* full = reinterpret_cast<uint64_t*>(wbest + CH_CONSUMER_WARPS);
    uint64_t* empty = full + CH_NB;
    int* s_token = reinterpret_cast<int*>(empty + CH_NB);
    MqLayerWeights* s_layers = reinterpret_cast<MqLayerWeights*>(s_token + 4);   // [num_layers]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int L = a.num_layers;

    Geometry ge;
    split_rows(QKV, cta, grid, ge.q0, ge.qn);
    split_rows(H, cta, grid, ge.o0, ge.on);
    split_rows(I, cta, grid, ge.g0, ge.gn);
    split_rows(a.vocab, cta, grid, ge.v0, ge.vn);
    ge.att_g = cta < NKV * a.nsplit ? cta / a.nsplit : -1;
    ge.att_s = cta < NKV * a.nsplit ? cta % a.nsplit : 0;

    if (tid == 0) {
        for (int i = 0; i < CH_NB; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], CH_CONSUMER_WARPS); }
        mbar_fence_init();
    }
    // the per-layer pointer table is read every phase: keep it in shared memory
    for (int i = tid; i < a.num_layers * (int)(sizeof(MqLayerWeights) / 8); i += CH_THREADS)
        reinterpret_cast<unsigned long long*>(s_layers)[i] = reinterpret_cast<const unsigned long long*>(a.layers)[i];
    __syncthreads();

    const uint32_t epoch0 = ld_relaxed_u32(a.epoch);
    const int pos0 = ld_cg_i32(a.pos0);
    const int n_lm_seg = (ge.vn + CH_LM_ROWS - 1) / CH_LM_ROWS;
    // tags: one per (step, layer), never 0
    auto tag32_of = [&](int step, int layer) { return epoch0 + (uint32_t)(step * (L + 1) + layer) + 1u; };
    auto tag16_of = [&](int step, int layer) { return ((epoch0 + (uint32_t)(step * (L + 1) + layer)) % 65535u) + 1u; };

    if (warp == CH_CONSUMER_WARPS) {
        // ============================================================ producer
        if (lane == 0) {
            // Ring space is tracked in "virtual" bytes: a piece that would cross the end of
            // the ring starts at the next lap instead, and piece k fits once its virtual end
            // is within one ring length of the oldest unreleased piece's virtual start.
            RingCursor rc{0u, 0u};
            uint32_t tail = 0;
            unsigned long long lap_base = 0ull;      // virtual position of ring offset 0 in the current lap
            unsigned long long v_start[CH_NB];
            bool dead = false;
            auto acquire = [&](uint32_t bytes, uint64_t*& bar) -> uint32_t {
                const uint32_t k = rc.seg;
                const uint32_t before = rc.head;
                const uint32_t off = rc.place(bytes);
                if (off == 0 && before != 0) lap_base += (unsigned long long)CH_RING_BYTES;
                const unsigned long long vs = lap_base + off, ve = vs + bytes;
                while (tail < k && ((k - tail) >= (uint32_t)CH_NB || ve - v_start[tail % CH_NB] > (unsigned long long)CH_RING_BYTES)) {
                    if (!dead && !mbar_wait(&empty[tail % CH_NB], (tail / CH_NB) & 1u, a.status)) dead = true;
                    ++tail;
                }
                v_start[k % CH_NB] = vs;
                bar = &full[k % CH_NB];
                mbar_expect_tx(bar, bytes);
                return off;
            };
            // pull the next layer's slices into L2 while this layer's go to shared memory
            auto prefetch_layer = [&](const MqLayerWeights& w) {
                int r = ge.q0;
                const int r1 = ge.q0 + ge.qn;
                while (r < r1) {
                    const bf16* base; int local, lim;
                    if (r < QSZ) { base = (const bf16*)w.q_proj; local = r; lim = QSZ; }
                    else if (r < QSZ + KVSZ) { base = (const bf16*)w.k_proj; local = r - QSZ; lim = QSZ + KVSZ; }
                    else { base = (const bf16*)w.v_proj; local = r - QSZ - KVSZ; lim = QKV; }
                    const int e = min(r1, lim);
                    l2_prefetch(base + (size_t)local * H, (uint32_t)(e - r) * H * 2);
                    r = e;
                }
                l2_prefetch((const bf16*)w.o_proj + (size_t)ge.o0 * QSZ, (uint32_t)ge.on * QSZ * 2);
                l2_prefetch((const bf16*)w.gate_proj + (size_t)ge.g0 * H, (uint32_t)ge.gn * H * 2);
                l2_prefetch((const bf16*)w.up_proj + (size_t)ge.g0 * H, (uint32_t)ge.gn * H * 2);
                l2_prefetch((const bf16*)w.down_proj + (size_t)ge.o0 * I, (uint32_t)ge.on * I * 2);
            };
            for (int step = 0; step < a.n_steps; ++step) {
                const int pos = pos0 + step;
                const AttPlan ap = att_plan(ge, pos, a.nsplit, (a.exp_flags & 4) != 0);
                for (int l = 0; l < L; ++l) {
                    const MqLayerWeights w = s_layers[l];
                    if (a.l2_ahead) {
                        if (l + 1 < L) prefetch_layer(s_layers[l + 1]);
                        else if (step + 1 < a.n_steps) prefetch_layer(s_layers[0]);
                    }
                    {   // input RMSNorm weight
                        uint64_t* bar;
                        const uint32_t off = acquire(H * 2, bar);
                        bulk_g2s(ring + off, w.input_layernorm, H * 2, bar);
                    }
                    // [Wq;Wk;Wv] rows
                    for (int p0 = 0; p0 < ge.qn; p0 += PR_QKV) {
                        const int rows = min(PR_QKV, ge.qn - p0);
                        uint64_t* bar;
                        const uint32_t off = acquire((uint32_t)rows * H * 2, bar);
                        int r = ge.q0 + p0;
                        const int r1 = r + rows;
                        while (r < r1) {
                            const bf16* base; int local, lim;
                            if (r < QSZ) { base = (const bf16*)w.q_proj; local = r; lim = QSZ; }
                            else if (r < QSZ + KVSZ) { base = (const bf16*)w.k_proj; local = r - QSZ; lim = QSZ + KVSZ; }
                            else { base = (const bf16*)w.v_proj; local = r - QSZ - KVSZ; lim = QKV; }
                            const int e = min(r1, lim);
                            bulk_g2s(ring + off + (size_t)(r - ge.q0 - p0) * H * 2, base + (size_t)local * H, (uint32_t)(e - r) * H * 2, bar);
                            r = e;
                        }
                    }
                    if (ap.active) {   // q_norm | k_norm | cos[pos] | sin[pos]
                        uint64_t* bar;
                        const uint32_t off = acquire(4 * D * 2, bar);
                        bulk_g2s(ring + off, w.q_norm, D * 2, bar);
                        bulk_g2s(ring + off + D * 2, w.k_norm, D * 2, bar);
                        bulk_g2s(ring + off + 2 * D * 2, a.cos + (size_t)pos * D, D * 2, bar);
                        bulk_g2s(ring + off + 3 * D * 2, a.sin + (size_t)pos * D, D * 2, bar);
                    }
                    if (ap.active && ap.n_cached > 0) {   // K chunk pieces, then V chunk pieces
                        const size_t head_off = ((size_t)(l * NKV + ge.att_g) * a.max_seq + ap.c0) * D;
                        // rows written by earlier steps of this launch were stored by other SMs, which
                        // fenced them (__threadfence) a full layer pass before this copy is issued
                        for (int kv = 0; kv < 2; ++kv)
                            for (int p0 = 0; p0 < ap.n_cached; p0 += PR_KV) {
                                const int rows = min(PR_KV, ap.n_cached - p0);
                                uint64_t* bar;
                                const uint32_t off = acquire((uint32_t)rows * D * 2, bar);
                                bulk_g2s(ring + off, (kv ? a.v_cache : a.k_cache) + head_off + (size_t)p0 * D, (uint32_t)rows * D * 2, bar);
                            }
                    }
                    for (int p0 = 0; p0 < ge.on; p0 += PR_O) {   // Wo rows
                        const int rows = min(PR_O, ge.on - p0);
                        uint64_t* bar;
                        const uint32_t off = acquire((uint32_t)rows * QSZ * 2, bar);
                        bulk_g2s(ring + off, (const bf16*)w.o_proj + (size_t)(ge.o0 + p0) * QSZ, (uint32_t)rows * QSZ * 2, bar);
                    }
                    {   // post-attention RMSNorm weight
                        uint64_t* bar;
                        const uint32_t off = acquire(H * 2, bar);
                        bulk_g2s(ring + off, w.post_attn_layernorm, H * 2, bar);
                    }
                    for (int p0 = 0; p0 < ge.gn; p0 += PR_GU) {  // gate rows then up rows of the same indices
                        const int rows = min(PR_GU, ge.gn - p0);
                        const uint32_t half = (uint32_t)rows * H * 2;
                        uint64_t* bar;
                        const uint32_t off = acquire(2 * half, bar);
                        bulk_g2s(ring + off, (const bf16*)w.gate_proj + (size_t)(ge.g0 + p0) * H, half, bar);
                        bulk_g2s(ring + off + half, (const bf16*)w.up_proj + (size_t)(ge.g0 + p0) * H, half, bar);
                    }
                    for (int p0 = 0; p0 < ge.on; p0 += PR_D) {   // Wd rows
                        const int rows = min(PR_D, ge.on - p0);
                        uint64_t* bar;
                        const uint32_t off = acquire((uint32_t)rows * I * 2, bar);
                        bulk_g2s(ring + off, (const bf16*)w.down_proj + (size_t)(ge.o0 + p0) * I, (uint32_t)rows * I * 2, bar);
                    }
                }
                {   // final RMSNorm weight
                    uint64_t* bar;
                    const uint32_t off = acquire(H * 2, bar);
                    bulk_g2s(ring + off, a.final_norm, H * 2, bar);
                }
                for (int sgi = 0; sgi < n_lm_seg; ++sgi) {   // LM-head rows
                    const int rows = min(CH_LM_ROWS, ge.vn - sgi * CH_LM_ROWS);
                    uint64_t* bar;
                    const uint32_t off = acquire((uint32_t)rows * H * 2, bar);
                    bulk_g2s(ring + off, a.lm_head + (size_t)(ge.v0 + sgi * CH_LM_ROWS) * H, (uint32_t)rows * H * 2, bar);
                }
            }
        }
        return;
    }

    // ============================================================== consumers
    const int ctid = tid;   // 0..255
    const size_t rofs = (size_t)(cta % CH_REP) * CH_XWORDS;   // this CTA's replica of the exchanged vectors
    const uint32_t* rxh = a.xh + rofs;
    const uint32_t* rxqkv = a.xqkv + rofs;
    const uint32_t* rxattn = a.xattn + rofs;
    const uint32_t* rxh1 = a.xh1 + rofs;
    const uint32_t* rxact = a.xact + rofs;
    Poller po{a.status, false, (a.exp_flags & 2) != 0};
    po.refresh();
    RingCursor rc{0u, 0u};
    int token = ld_cg_i32(a.first_token);
    if (cta == 0 && ctid == 0) {
        if (token < 0 || token >= a.vocab) atomicOr(a.status, MQ_STATUS_BAD_TOKEN);
        if (pos0 < 0 || pos0 + a.n_steps > a.max_seq) atomicOr(a.status, MQ_STATUS_BAD_POSITION);
    }
    token = min(max(token, 0), a.vocab - 1);
    float resid = 0.f;   // residual stream of row o0 + ctid (threads < on)
    int xsel = 0;

    auto piece_wait = [&](const Pieces& P, int p) {
        const uint32_t k = P.k0 + (uint32_t)p;
        mbar_wait(&full[k % CH_NB], (k / CH_NB) & 1u, a.status);
    };
    auto single_wait = [&](uint32_t bytes, uint32_t& k) -> uint32_t {
        k = rc.seg;
        const uint32_t off = rc.place(bytes);
        mbar_wait(&full[k % CH_NB], (k / CH_NB) & 1u, a.status);
        return off;
    };
    auto single_release = [&](uint32_t k) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[k % CH_NB]);
    };
    auto pieces_release = [&](const Pieces& P) {
        __syncwarp();
        if (lane == 0)
            for (int p = 0; p < P.np; ++p) mbar_arrive(&empty[(P.k0 + (uint32_t)p) % CH_NB]);
    };
    // stage timers (thread 0 of each CTA): 0 poll A, 1 poll B, 2 poll C, 3 poll D, 4 poll E, 5 weights, 6 lm, 7 total
    // accumulated in shared memory so that they cost no registers
    unsigned long long* tacc = reinterpret_cast<unsigned long long*>(s_layers + CH_MAX_LAYERS);   // [16]
    unsigned long long* ttrace = tacc + 16;   // [64] phase time stamps of step 2, layers 0..2 (cycles since the step began)
    if (ctid == 0) for (int i = 0; i < 80; ++i) tacc[i] = 0ull;
    long long t_step = 0;
    const bool timing = a.dbg != nullptr && ctid == 0;
    const long long t_begin = clock64();
#define TRACE(i) do { if (timing && step == 20 && l >= 10 && l < 13) ttrace[(l - 10) * 20 + (i)] = (unsigned long long)(clock64() - t_step); } while (0)
#define TSTART() long long _t0 = timing ? clock64() : 0
#ifdef MQ_CHAIN_FINE_TIMERS
#define TSTART2() long long _t1 = timing ? clock64() : 0
#define TSTOP2(i) do { if (timing) tacc[i] += (unsigned long long)(clock64() - _t1); } while (0)
#else
#define TSTART2() do { } while (0)
#define TSTOP2(i) do { } while (0)
#endif
#define TSTOP(i) do { if (timing) tacc[i] += (unsigned long long)(clock64() - _t0); } while (0)

    if (a.exp_flags & 8) {
        // experiment: consumers only wait for and release every ring piece (pure stream rate)
        auto drain = [&](int rows, int pr, uint32_t row_bytes) {
            const Pieces P = place_pieces(rc, rows, pr, row_bytes);
            for (int p = 0; p < P.np; ++p) piece_wait(P, p);
            pieces_release(P);
        };
        for (int step = 0; step < a.n_steps; ++step) {
            for (int l = 0; l < L; ++l) {
                uint32_t k;
                single_wait(H * 2, k); single_release(k);
                drain(ge.qn, PR_QKV, H * 2);
                drain(ge.on, PR_O, QSZ * 2);
                single_wait(H * 2, k); single_release(k);
                drain(ge.gn, PR_GU, 2 * H * 2);
                drain(ge.on, PR_D, I * 2);
            }
            uint32_t k;
            single_wait(H * 2, k); single_release(k);
            for (int sgi = 0; sgi < n_lm_seg; ++sgi) {
                const int rows = min(CH_LM_ROWS, ge.vn - sgi * CH_LM_ROWS);
                single_wait((uint32_t)rows * H * 2, k); single_release(k);
            }
            if (cta == 0 && ctid == 0) a.tokens_out[step] = 0;
        }
        if (cta == 0 && ctid == 0) st_relaxed_u32(a.epoch, epoch0 + (uint32_t)(a.n_steps * (L + 1)));
        return;
    }
    for (int step = 0; step < a.n_steps; ++step) {
        const int pos = pos0 + step;
        const AttPlan ap = att_plan(ge, pos, a.nsplit, (a.exp_flags & 4) != 0);
        if (ctid < ge.on) resid = bf2f(a.embed[(size_t)token * H + ge.o0 + ctid]);
        if (timing && step == 20) t_step = clock64();

        for (int l = 0; l < L; ++l) {
            const MqLayerWeights w = s_layers[l];
            const uint32_t t16 = tag16_of(step, l), t32 = tag32_of(step, l);
            float x[32];

            // ---------------- phase A: RMSNorm + QKV rows
            TRACE(0);
            {
                bf16* xb = xbuf + xsel * I; xsel ^= 1;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                const bool has = ctid < H / 4;
                if (l == 0) {
                    if (has) {
                        const uint2 u = __ldg(reinterpret_cast<const uint2*>(a.embed + (size_t)token * H + 4 * ctid));
                        v[0] = bf_lo(u.x); v[1] = bf_hi(u.x); v[2] = bf_lo(u.y); v[3] = bf_hi(u.y);
                    }
                } else {
                    TSTART();
                    if (has) {
                        const uint4 u = po.words4(rxh + 4 * ctid, tag16_of(step, l - 1));
                        v[0] = bf_hi(u.x); v[1] = bf_hi(u.y); v[2] = bf_hi(u.z); v[3] = bf_hi(u.w);
                    }
                    TSTOP(0);
                }
                TSTART2();
                uint32_t kn;
                const uint32_t noff = single_wait(H * 2, kn);
                coop_rmsnorm_store(v, has, reinterpret_cast<const bf16*>(ring + noff), xb, red, ctid, lane, warp);
                single_release(kn);
                load_x_smem<4>(x, xb, lane);
                TSTOP2(13);
                TRACE(1);
            }
            {
                TSTART2();
                const Pieces P = place_pieces(rc, ge.qn, PR_QKV, H * 2);
                const bf16* rows[4];
                bool ok[4];
                int idx[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    idx[r] = warp + r * CH_CONSUMER_WARPS;
                    ok[r] = idx[r] < ge.qn && !(a.exp_flags & 1);
                    rows[r] = reinterpret_cast<const bf16*>(ring);
                    if (ok[r]) {
                        { TSTART(); piece_wait(P, idx[r] / PR_QKV); TSTOP(5); }
                        rows[r] = reinterpret_cast<const bf16*>(ring + piece_off(P, idx[r] / PR_QKV)) + (size_t)(idx[r] % PR_QKV) * H;
                    }
                }
                float d[4];
                dots_multi<4, 4>(rows, ok, x, lane, d);
                if (lane < 4) {
                    const float dv = lane == 0 ? d[0] : (lane == 1 ? d[1] : (lane == 2 ? d[2] : d[3]));
                    const int i = warp + lane * CH_CONSUMER_WARPS;
                    if (i < ge.qn) publish(a.xqkv, ge.q0 + i, rbf(dv), t16);
                }
                pieces_release(P);
                TSTOP2(8);
                TRACE(2);
            }

            // ---------------- phase B: attention item (g, s)
            if (ap.active) {
                TSTART2();
                const int g = ge.att_g, n = ap.n;
                bf16* xb = xbuf + xsel * I; xsel ^= 1;
                // raw q(2g), q(2g+1), k(g), v(g): 4 x 128 words
                {
                    TSTART();
                    if (ctid < 128) {
                        const int which = ctid >> 5, c = ctid & 31;
                        const int base = which < 2 ? (2 * g + which) * D : (which == 2 ? QSZ + g * D : QSZ + KVSZ + g * D);
                        const uint4 v = po.words4(rxqkv + base + 4 * c, t16);
                        uint2 o;
                        o.x = (v.x >> 16) | (v.y & 0xffff0000u);
                        o.y = (v.z >> 16) | (v.w & 0xffff0000u);
                        *reinterpret_cast<uint2*>(xb + which * D + 4 * c) = o;
                    }
                    consumer_bar();
                    TSTOP(1);
                }
                TRACE(3);
                // constants piece (q_norm | k_norm | cos | sin), then K and V pieces: placed now to
                // keep the cursor in step with the producer, waited for where they are needed
                const uint32_t kc = rc.seg;
                const uint32_t coff = rc.place(4 * D * 2);
                Pieces PK, PV;
                PK.np = PV.np = 0; PK.k0 = PV.k0 = 0;
                if (ap.n_cached > 0) {
                    PK = place_pieces(rc, ap.n_cached, PR_KV, D * 2);
                    PV = place_pieces(rc, ap.n_cached, PR_KV, D * 2);
                }
                bf16* krow = xb + 4 * D;           // new position's K (after norm + RoPE)
                bf16* vrow = xb + 5 * D;           // new position's V
                const bf16* cst = reinterpret_cast<const bf16*>(ring + coff);
                const bf16* cosr = cst + 2 * D;
                const bf16* sinr = cst + 3 * D;
                const size_t head_off = ((size_t)(l * NKV + g) * a.max_seq) * D;
                mbar_wait(&full[kc % CH_NB], (kc / CH_NB) & 1u, a.status);
                if (warp < 2) {
                    float lo[2], hi[2];
                    norm_rope_smem(xb + warp * D, cst, cosr, sinr, lane, lo, hi);
                    qh[warp * D + 2 * lane] = lo[0]; qh[warp * D + 2 * lane + 1] = lo[1];
                    qh[warp * D + 64 + 2 * lane] = hi[0]; qh[warp * D + 64 + 2 * lane + 1] = hi[1];
                } else if (warp == 2 && ap.is_last) {
                    float lo[2], hi[2];
                    norm_rope_smem(xb + 2 * D, cst + D, cosr, sinr, lane, lo, hi);
                    const uint32_t plo = pack_bf16x2(lo[0], lo[1]), phi = pack_bf16x2(hi[0], hi[1]);
                    *reinterpret_cast<uint32_t*>(krow + 2 * lane) = plo;
                    *reinterpret_cast<uint32_t*>(krow + 64 + 2 * lane) = phi;
                    bf16* gk = a.k_cache + head_off + (size_t)pos * D;
                    *reinterpret_cast<uint32_t*>(gk + 2 * lane) = plo;
                    *reinterpret_cast<uint32_t*>(gk + 64 + 2 * lane) = phi;
                } else if (warp == 3 && ap.is_last) {
                    const uint2 u = *reinterpret_cast<const uint2*>(xb + 3 * D + 4 * lane);
                    *reinterpret_cast<uint2*>(vrow + 4 * lane) = u;
                    *reinterpret_cast<uint2*>(a.v_cache + head_off + (size_t)pos * D + 4 * lane) = u;
                }
                single_release(kc);
                consumer_bar();
                TRACE(4);
                // scores: 8 lanes per position, 4 positions per warp pass
                {
                    const int psub = lane >> 3, prt = lane & 7;
                    float q0[16], q1[16];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        q0[e] = qh[prt * 8 + e]; q0[8 + e] = qh[64 + prt * 8 + e];
                        q1[e] = qh[D + prt * 8 + e]; q1[8 + e] = qh[D + 64 + prt * 8 + e];
                    }
                    const float scale = 0.08838834764831845f;
                    for (int p4 = warp * 4; p4 < n; p4 += CH_CONSUMER_WARPS * 4) {
                        const int p = p4 + psub;
                        float s0 = 0.f, s1 = 0.f;
                        if (p4 < ap.n_cached) { TSTART(); piece_wait(PK, p4 / PR_KV); TSTOP(5); }   // 4 | PR_KV: one piece per pass
                        if (p < n) {
                            const bf16* rowp = (p < ap.n_cached)
                                ? reinterpret_cast<const bf16*>(ring + piece_off(PK, p / PR_KV)) + (size_t)(p % PR_KV) * D : krow;
                            const uint4 ua = *reinterpret_cast<const uint4*>(rowp + prt * 8);
                            const uint4 ub = *reinterpret_cast<const uint4*>(rowp + 64 + prt * 8);
                            const float kv[16] = {bf_lo(ua.x), bf_hi(ua.x), bf_lo(ua.y), bf_hi(ua.y), bf_lo(ua.z), bf_hi(ua.z), bf_lo(ua.w), bf_hi(ua.w),
                                                  bf_lo(ub.x), bf_hi(ub.x), bf_lo(ub.y), bf_hi(ub.y), bf_lo(ub.z), bf_hi(ub.z), bf_lo(ub.w), bf_hi(ub.w)};
#pragma unroll
                            for (int e = 0; e < 16; ++e) { s0 = fmaf(kv[e], q0[e], s0); s1 = fmaf(kv[e], q1[e], s1); }
                        }
#pragma unroll
                        for (int o = 4; o > 0; o >>= 1) {
                            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                        }
                        if (prt == 0 && p < n) { sc[p] = s0 * scale; sc[CH_MAX_CAP + p] = s1 * scale; }
                    }
                }
                if (ap.n_cached > 0) pieces_release(PK);
                consumer_bar();
                TRACE(5);
                if (warp < 2) {
                    float* srow = sc + warp * CH_MAX_CAP;
                    float m = -INFINITY;
                    for (int p = lane; p < n; p += 32) m = fmaxf(m, srow[p]);
                    m = warp_max(m);
                    float lsum = 0.f;
                    for (int p = lane; p < n; p += 32) {
                        const float e = expf(srow[p] - m);
                        lsum += e;
                        srow[p] = rbf(e);
                    }
                    lsum = warp_sum(lsum);
                    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = lsum; }
                }
                consumer_bar();
                TRACE(6);
                {   // PV: thread = (head, half of the positions, pair of dims)
                    const int hh = ctid >> 7, third = (ctid >> 6) & 1, dp = ctid & 63;   // two halves of the positions
                    const int nt = (n + 1) / 2;
                    const int pb = third * nt, pe = min(n, pb + nt);
                    const float* prow = sc + hh * CH_MAX_CAP;
                    float a0 = 0.f, a1 = 0.f;
                    int waited = -1;
                    for (int p = pb; p < pe; ++p) {
                        const bf16* rowp = vrow;
                        if (p < ap.n_cached) {
                            const int pc = p / PR_KV;
                            if (pc != waited) { piece_wait(PV, pc); waited = pc; }
                            rowp = reinterpret_cast<const bf16*>(ring + piece_off(PV, pc)) + (size_t)(p % PR_KV) * D;
                        }
                        const uint32_t u = *reinterpret_cast<const uint32_t*>(rowp + 2 * dp);
                        const float pv = prow[p];
                        a0 = fmaf(pv, bf_lo(u), a0);
                        a1 = fmaf(pv, bf_hi(u), a1);
                    }
                    accb[(hh * 2 + third) * D + 2 * dp] = a0;
                    accb[(hh * 2 + third) * D + 2 * dp + 1] = a1;
                }
                if (ap.n_cached > 0) pieces_release(PV);
                consumer_bar();
                TRACE(7);
                if (ctid < 2 * D) {
                    const int hh = ctid >> 7, d = ctid & 127;
                    const float acc = accb[(hh * 2) * D + d] + accb[(hh * 2 + 1) * D + d];
                    const int qhead = 2 * g + hh;
                    if (ap.n_act == 1) {
                        publish(a.xattn, qhead * D + d, rbf(acc / ml[hh * 2 + 1]), t16);
                    } else {
                        const size_t pbase = ((size_t)qhead * a.nsplit + ge.att_s) * CH_PART;
                        publish_f32(a.xpart, pbase + 2 + d, acc, t32);
                        if (d == 0) {
                            publish_f32(a.xpart, pbase, ml[hh * 2], t32);
                            publish_f32(a.xpart, pbase + 1, ml[hh * 2 + 1], t32);
                        }
                        if (ge.att_s == 0) {   // this CTA merges the splits of its two heads
                            // (m, l) of split `lane`, one round trip for the whole warp
                            float mj = -INFINITY, lj = 0.f;
                            if (lane < ap.n_act) {
                                const unsigned long long* pj = a.xpart + ((size_t)qhead * a.nsplit + lane) * CH_PART;
                                mj = po.f32(pj, t32);
                                lj = po.f32(pj + 1, t32);
                            }
                            const float M = warp_max(mj);
                            const float fj = (lane < ap.n_act) ? expf(mj - M) : 0.f;
                            const float den = warp_sum(lj * fj);
                            // acc[d] of every split: all loads issued before the first tag check
                            unsigned long long raw[CH_MAX_SPLIT];
#pragma unroll
                            for (int j = 0; j < CH_MAX_SPLIT; ++j)
                                if (j < ap.n_act) raw[j] = ld_relaxed_u64(a.xpart + ((size_t)qhead * a.nsplit + j) * CH_PART + 2 + d);
                            float num = 0.f;
#pragma unroll
                            for (int j = 0; j < CH_MAX_SPLIT; ++j) {
                                const float f = __shfl_sync(0xffffffffu, fj, j);
                                if (j < ap.n_act) {
                                    float v = __uint_as_float((uint32_t)raw[j]);
                                    if ((uint32_t)(raw[j] >> 32) != t32)
                                        v = po.f32(a.xpart + ((size_t)qhead * a.nsplit + j) * CH_PART + 2 + d, t32);
                                    num = fmaf(v, f, num);
                                }
                            }
                            publish(a.xattn, qhead * D + d, rbf(num / den), t16);
                        }
                    }
                }
                if (ap.is_last) __threadfence();   // new K/V rows must be visible to later bulk copies
                TSTOP2(9);
                TRACE(8);
            }

            // ---------------- phase C: Wo rows + residual
            {
                bf16* xb = xbuf + xsel * I; xsel ^= 1;
                TRACE(9);
                { TSTART(); poll_vector(po, rxattn, QSZ, t16, xb, ctid); consumer_bar(); TSTOP(2); }
                TRACE(10);
                TSTART2();
                const int half = warp & 1;
                load_x_smem<4>(x, xb + half * 1024, lane);
                const Pieces P = place_pieces(rc, ge.on, PR_O, QSZ * 2);
                const bf16* rows[2];
                bool ok[2];
                int idx[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    idx[r] = (warp >> 1) + r * (CH_CONSUMER_WARPS / 2);
                    ok[r] = idx[r] < ge.on && !(a.exp_flags & 1);
                    rows[r] = reinterpret_cast<const bf16*>(ring);
                    if (ok[r]) {
                        { TSTART(); piece_wait(P, idx[r] / PR_O); TSTOP(5); }
                        rows[r] = reinterpret_cast<const bf16*>(ring + piece_off(P, idx[r] / PR_O)) + (size_t)(idx[r] % PR_O) * QSZ + half * 1024;
                    }
                }
                float d[2];
                dots_multi<2, 4>(rows, ok, x, lane, d);
                if (lane < 2) {
                    const int r = (warp >> 1) + lane * (CH_CONSUMER_WARPS / 2);
                    if (r < ge.on) part[r * 4 + half] = lane == 0 ? d[0] : d[1];
                }
                pieces_release(P);
                consumer_bar();
                if (ctid < ge.on) {
                    const float o = rbf(part[ctid * 4] + part[ctid * 4 + 1]);
                    resid = rbf(resid + o);
                    publish(a.xh1, ge.o0 + ctid, resid, t16);
                }
                TSTOP2(10);
                TRACE(11);
            }

            // ---------------- phase D: RMSNorm + gate/up rows + SiLU*up
            {
                bf16* xb = xbuf + xsel * I; xsel ^= 1;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                const bool has = ctid < H / 4;
                {
                    TSTART();
                    if (has) {
                        const uint4 u = po.words4(rxh1 + 4 * ctid, t16);
                        v[0] = bf_hi(u.x); v[1] = bf_hi(u.y); v[2] = bf_hi(u.z); v[3] = bf_hi(u.w);
                    }
                    TSTOP(3);
                }
                TSTART2();
                uint32_t kn;
                const uint32_t noff = single_wait(H * 2, kn);
                coop_rmsnorm_store(v, has, reinterpret_cast<const bf16*>(ring + noff), xb, red, ctid, lane, warp);
                single_release(kn);
                load_x_smem<4>(x, xb, lane);
                TRACE(12);
                const Pieces P = place_pieces(rc, ge.gn, PR_GU, 2 * H * 2);
                // pairs i = warp, warp + 8, warp + 16: rows {gate_i, up_i} x 3
                const bf16* rows[6];
                bool ok[6];
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const int i = warp + r * CH_CONSUMER_WARPS;
                    ok[2 * r] = ok[2 * r + 1] = i < ge.gn && !(a.exp_flags & 1);
                    rows[2 * r] = rows[2 * r + 1] = reinterpret_cast<const bf16*>(ring);
                    if (i < ge.gn) {
                        const int pc = i / PR_GU, prow = min(PR_GU, ge.gn - pc * PR_GU);
                        { TSTART(); piece_wait(P, pc); TSTOP(5); }
                        const bf16* gb = reinterpret_cast<const bf16*>(ring + piece_off(P, pc));
                        rows[2 * r] = gb + (size_t)(i % PR_GU) * H;
                        rows[2 * r + 1] = gb + (size_t)prow * H + (size_t)(i % PR_GU) * H;
                    }
                }
                float d[6];
                dots_multi<6, 4>(rows, ok, x, lane, d);
                if (lane < 3) {
                    const int i = warp + lane * CH_CONSUMER_WARPS;
                    if (i < ge.gn) {
                        const float gs = lane == 0 ? d[0] : (lane == 1 ? d[2] : d[4]);
                        const float us = lane == 0 ? d[1] : (lane == 1 ? d[3] : d[5]);
                        const float act = rbf(silu_f32(rbf(gs)));
                        publish(a.xact, ge.g0 + i, rbf(act * rbf(us)), t16);
                    }
                }
                pieces_release(P);
                TSTOP2(11);
                TRACE(13);
            }

            // ---------------- phase E: Wd rows + residual
            {
                bf16* xb = xbuf + xsel * I; xsel ^= 1;
                { TSTART(); poll_vector(po, rxact, I, t16, xb, ctid); consumer_bar(); TSTOP(4); }
                TRACE(14);
                TSTART2();
                // K = 3072 in four quarters of 768 columns: warp = (row group, quarter)
                const int quarter = warp & 3;
                float xq[24];
                load_x_smem<3>(xq, xb + quarter * 768, lane);
                const Pieces P = place_pieces(rc, ge.on, PR_D, I * 2);
                const bf16* rows[4];
                bool ok[4];
                int idx[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    idx[r] = (warp >> 2) + 2 * r;
                    ok[r] = idx[r] < ge.on && !(a.exp_flags & 1);
                    rows[r] = reinterpret_cast<const bf16*>(ring);
                    if (ok[r]) {
                        { TSTART(); piece_wait(P, idx[r] / PR_D); TSTOP(5); }
                        rows[r] = reinterpret_cast<const bf16*>(ring + piece_off(P, idx[r] / PR_D)) + (size_t)(idx[r] % PR_D) * I + quarter * 768;
                    }
                }
                float d[4];
                dots_multi<4, 3>(rows, ok, xq, lane, d);
                if (lane < 4) {
                    const int r = (warp >> 2) + 2 * lane;
                    if (r < ge.on) part[r * 4 + quarter] = lane == 0 ? d[0] : (lane == 1 ? d[1] : (lane == 2 ? d[2] : d[3]));
                }
                pieces_release(P);
                consumer_bar();
                if (ctid < ge.on) {
                    const float dn = rbf(part[ctid * 4] + part[ctid * 4 + 1] + part[ctid * 4 + 2] + part[ctid * 4 + 3]);
                    resid = rbf(resid + dn);
                    publish(a.xh, ge.o0 + ctid, resid, t16);
                }
                TSTOP2(12);
                TRACE(15);
            }
        }

        // ---------------- LM head + arg-max, result known to every CTA
        {
            TSTART();
            float x[32];
            bf16* xb = xbuf + xsel * I; xsel ^= 1;
            {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                const bool has = ctid < H / 4;
                if (has) {
                    const uint4 u = po.words4(rxh + 4 * ctid, tag16_of(step, L - 1));
                    v[0] = bf_hi(u.x); v[1] = bf_hi(u.y); v[2] = bf_hi(u.z); v[3] = bf_hi(u.w);
                }
                uint32_t kn;
                const uint32_t noff = single_wait(H * 2, kn);
                coop_rmsnorm_store(v, has, reinterpret_cast<const bf16*>(ring + noff), xb, red, ctid, lane, warp);
                single_release(kn);
                load_x_smem<4>(x, xb, lane);
            }
            float bestv = -INFINITY;
            int besti = 0x7fffffff;
            const bool want_logits = a.logits != nullptr && step == a.n_steps - 1;
            for (int sgi = 0; sgi < n_lm_seg; ++sgi) {
                const int rows = min(CH_LM_ROWS, ge.vn - sgi * CH_LM_ROWS);
                const uint32_t k = rc.seg;
                const uint32_t off = rc.place((uint32_t)rows * H * 2);
                mbar_wait(&full[k % CH_NB], (k / CH_NB) & 1u, a.status);
                {
                    const bf16* sb = reinterpret_cast<const bf16*>(ring + off);
                    const bf16* rows2[2] = {sb + (size_t)warp * H, sb + (size_t)(warp + CH_CONSUMER_WARPS) * H};
                    const bool ok2[2] = {warp < rows, warp + CH_CONSUMER_WARPS < rows};
                    float dv[2];
                    dots_multi<2, 4>(rows2, ok2, x, lane, dv);
                    if (lane == 0) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            if (ok2[r]) {
                                const float lv = rbf(dv[r]);
                                const int gi = ge.v0 + sgi * CH_LM_ROWS + warp + r * CH_CONSUMER_WARPS;
                                if (want_logits) a.logits[gi] = lv;
                                if (lv > bestv) { bestv = lv; besti = gi; }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[k % CH_NB]);
            }
            const uint32_t t32 = tag32_of(step, L);
            if (lane == 0) {
                uint32_t u = __float_as_uint(bestv);
                u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                wbest[warp] = (besti == 0x7fffffff) ? 0ull : (((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)besti));
            }
            consumer_bar();
            if (ctid == 0) {
                unsigned long long kbest = 0ull;
                for (int i = 0; i < CH_CONSUMER_WARPS; ++i) kbest = wbest[i] > kbest ? wbest[i] : kbest;
                st_relaxed_u64(a.xlm + 2 * cta, ((unsigned long long)t32 << 32) | (kbest >> 32));
                st_relaxed_u64(a.xlm + 2 * cta + 1, ((unsigned long long)t32 << 32) | (kbest & 0xffffffffull));
            }
            // every CTA gathers all per-CTA maxima and reduces them itself
            unsigned long long mine = 0ull;
            for (int c = ctid; c < grid; c += CH_CONSUMERS) {
                const uint32_t hi = __float_as_uint(po.f32(a.xlm + 2 * c, t32));
                const uint32_t lo = __float_as_uint(po.f32(a.xlm + 2 * c + 1, t32));
                const unsigned long long kc = ((unsigned long long)hi << 32) | lo;
                mine = kc > mine ? kc : mine;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
                mine = other > mine ? other : mine;
            }
            consumer_bar();            // wbest reads above are done
            if (lane == 0) wbest[warp] = mine;
            consumer_bar();
            if (ctid == 0) {
                unsigned long long kbest = 0ull;
                for (int i = 0; i < CH_CONSUMER_WARPS; ++i) kbest = wbest[i] > kbest ? wbest[i] : kbest;
                const int tk = (int)(0xffffffffu - (uint32_t)(kbest & 0xffffffffull));
                *s_token = min(max(tk, 0), a.vocab - 1);
                if (cta == 0) a.tokens_out[step] = *s_token;
            }
            consumer_bar();
            token = *s_token;
            TSTOP(6);
        }
    }
    if (timing) {
        tacc[7] = (unsigned long long)(clock64() - t_begin);
        for (int i = 0; i < 80; ++i) a.dbg[(size_t)cta * 80 + i] = tacc[i];
    }
#undef TSTART
#undef TRACE
#undef TSTART2
#undef TSTOP2
#undef TSTOP
    // The last exchange above needed data from every CTA, so every CTA has long
    // since read the old epoch: advancing it here is race-free.
    if (cta == 0 && ctid == 0) st_relaxed_u32(a.epoch, epoch0 + (uint32_t)(a.n_steps * (L + 1)));
}

static size_t chain_smem_bytes() {
    return (size_t)CH_RING_BYTES + 2 * I * 2 + (2 * CH_MAX_CAP + 2 * D + 6 * D + 4 + 32 + 16) * 4 + CH_CONSUMER_WARPS * 8 + 2 * CH_NB * 8 + 16 + CH_MAX_LAYERS * sizeof(MqLayerWeights) + 16 * 8 + 64 * 8;
}

static int chain_nsplit(int max_seq) {
    int ns = (max_seq + 127) / 128;
    return ns < 1 ? 1 : (ns > CH_MAX_SPLIT ? CH_MAX_SPLIT : ns);
}

struct ChainDevice {
    bool ready = false;
    int sm_count = 0;
};
static ChainDevice g_chain_dev[64];

static int chain_ensure(ChainDevice** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
    ChainDevice& st = g_chain_dev[dev];
    if (!st.ready) {
        cudaDeviceProp p;
        e = cudaGetDeviceProperties(&p, dev);
        if (e != cudaSuccess) return (int)e;
        if (p.major != 10 || p.multiProcessorCount < CH_MIN_GRID || !p.cooperativeLaunch) return MQ_ERR_UNSUPPORTED;
        st.sm_count = p.multiProcessorCount;
        e = cudaFuncSetAttribute(k_decode_chain, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)chain_smem_bytes());
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_chain, CH_THREADS, chain_smem_bytes());
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return MQ_ERR_UNSUPPORTED;
        st.ready = true;
    }
    *out = &st;
    return MQ_OK;
}

}  // namespace mq

using namespace mq;

// Tuning / instrumentation knobs (process-wide; meant for benchmarks and tests).
static unsigned long long* g_chain_dbg = nullptr;
static int g_chain_l2_ahead = 1;

extern "C" int mq_chain_set_debug(unsigned long long* stage_cycles_dev, int l2_prefetch_ahead) {
    g_chain_dbg = stage_cycles_dev;
    g_chain_l2_ahead = l2_prefetch_ahead;   // bit 0: L2 prefetch; bits 8+: experiment flags
    return MQ_OK;
}

extern "C" int mq_chain_init_device(void) {
    ChainDevice* st = nullptr;
    return chain_ensure(&st);
}

extern "C" int mq_chain_max_seq_len(void) { return CH_MAX_SPLIT * CH_MAX_CAP; }

extern "C" size_t mq_chain_scratch_bytes(void) {
    // tagged vectors + split partials + per-CTA maxima + epoch word, each 256-byte aligned
    size_t n = 0;
    n += (size_t)CH_REP * CH_XWORDS * 4;
    n = (n + 255) & ~(size_t)255;
    n += (size_t)NQ * CH_MAX_SPLIT * CH_PART * 8;
    n = (n + 255) & ~(size_t)255;
    n += (size_t)2 * 256 * 8;
    n += 256;
    return n;
}

extern "C" int mq_launch_decode_chain(const MqModel* model, const MqLayerWeights* layers_dev, void* k_cache, void* v_cache,
                                      void* scratch, unsigned int* status, const int* first_token, const int* position0,
                                      int* tokens_out, int n_steps, float* last_logits, void* stream_v) {
    if (!model || !layers_dev || !k_cache || !v_cache || !scratch || !status || !first_token || !position0 || !tokens_out)
        return MQ_ERR_BAD_ARG;
    if (n_steps <= 0 || model->num_layers <= 0 || model->vocab_size <= 0 || model->max_seq_len <= 0) return MQ_ERR_BAD_ARG;
    if (model->max_seq_len > CH_MAX_SPLIT * CH_MAX_CAP) return MQ_ERR_TOO_LONG;
    if (model->num_layers > CH_MAX_LAYERS) return MQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(scratch) & 255u) || (reinterpret_cast<uintptr_t>(k_cache) & 15u) ||
        (reinterpret_cast<uintptr_t>(v_cache) & 15u) || (reinterpret_cast<uintptr_t>(model->lm_head) & 15u))
        return MQ_ERR_ALIGNMENT;
    ChainDevice* st = nullptr;
    int rc = chain_ensure(&st);
    if (rc != MQ_OK) return rc;
    if (st->sm_count > 256) return MQ_ERR_UNSUPPORTED;
    if (model->vocab_size < st->sm_count) return MQ_ERR_BAD_ARG;

    ChainArgs a;
    a.embed = (const bf16*)model->embed;
    a.final_norm = (const bf16*)model->final_norm;
    a.lm_head = (const bf16*)model->lm_head;
    a.cos = (const bf16*)model->cos_table;
    a.sin = (const bf16*)model->sin_table;
    a.layers = layers_dev;
    a.k_cache = (bf16*)k_cache;
    a.v_cache = (bf16*)v_cache;
    uint8_t* s = static_cast<uint8_t*>(scratch);
    a.xh = reinterpret_cast<uint32_t*>(s);
    a.xqkv = a.xh + H;
    a.xattn = a.xqkv + QKV;
    a.xh1 = a.xattn + QSZ;
    a.xact = a.xh1 + H;
    size_t off = ((size_t)CH_REP * CH_XWORDS * 4 + 255) & ~(size_t)255;
    a.xpart = reinterpret_cast<unsigned long long*>(s + off);
    off = (off + (size_t)NQ * CH_MAX_SPLIT * CH_PART * 8 + 255) & ~(size_t)255;
    a.xlm = reinterpret_cast<unsigned long long*>(s + off);
    off += (size_t)2 * 256 * 8;
    a.epoch = reinterpret_cast<uint32_t*>(s + off);
    a.status = status;
    a.first_token = first_token;
    a.pos0 = position0;
    a.tokens_out = tokens_out;
    a.logits = last_logits;
    a.dbg = g_chain_dbg;
    a.l2_ahead = g_chain_l2_ahead & 1;
    a.exp_flags = g_chain_l2_ahead >> 8;
    a.num_layers = model->num_layers;
    a.vocab = model->vocab_size;
    a.max_seq = model->max_seq_len;
    a.n_steps = n_steps;
    a.nsplit = chain_nsplit(model->max_seq_len);
    a.chunk_cap = CH_MAX_CAP;

    void* params[] = {&a};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)k_decode_chain, dim3(st->sm_count), dim3(CH_THREADS), params,
                                                chain_smem_bytes(), (cudaStream_t)stream_v);
    return (int)e;
}
