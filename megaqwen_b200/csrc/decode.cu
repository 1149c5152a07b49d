// Batch-1 greedy decode step for sm_100a: six weight-streaming kernels per
// token position chained with programmatic dependent launch (PDL).
//
// Design.  One decode step is HBM-bound (1.19 GB of bf16 weights + the KV
// cache per token) but consists of ~140 dependent phases.  Instead of a
// cooperative grid with a grid-wide barrier per phase (the reference:
// csrc/megakernel/fused_decode_ldg_kernel.inl:43-137, 225 grid.sync() calls)
// every phase is its own kernel of one CTA per SM, and every kernel starts with
// a prologue that does not depend on the previous phase: it pulls the CTA's
// whole slice of the weight matrix (contiguous rows, 28-96 KB) into shared
// memory with 1-D TMA bulk copies, then executes griddepcontrol.wait.  Because
// each kernel releases its dependents at once, the weight stream of phase n+1
// (and n+2, shared memory permitting) overlaps the arithmetic and the drain of
// phase n, and the hardware tracks the dependency: no flag spinning anywhere.
//
// Rounding points follow the HuggingFace bf16 model (bf16 out of every linear,
// norm, RoPE product and sum, activation, product and residual add; fp32
// accumulation inside dot products, norms and softmax).
//
// Phases per layer (reference stage each one replaces):
//   k_qkv     RMSNorm + [Wq;Wk;Wv] GEMV        fused_decode_ldg_common.inl:131-262
//   k_attn    QK-norm + RoPE + cache write + split-KV GQA attention
//                                              fused_decode_ldg_common.inl:268-394, 417-794
//   k_oproj   Wo GEMV + residual               fused_decode_ldg_mlp.inl:5-63
//   k_gateup  RMSNorm + gate/up GEMV + SiLU*up fused_decode_ldg_mlp.inl:64-170
//   k_down    Wd GEMV + residual               fused_decode_ldg_mlp.inl:171-218
// then k_lmhead: final RMSNorm + tied LM head + arg-max
//                                              fused_decode_ldg_kernel.inl:104-137, fused_decode_ldg_lm.inl:6-163
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mq_device.cuh"

namespace mq {

// The experiment switches cost registers and branches in every kernel, so they are
// compiled in only with -DMQ_DECODE_EXPERIMENTS.
#ifdef MQ_DECODE_EXPERIMENTS
#define EXPF(a) ((a).exp_flags)
#else
#define EXPF(a) 0
#endif

// Timeline builds (-DMQ_TIMELINE) stamp %globaltimer at entry (0), after the dependency
// wait (1), before the dot products (2) and at the end (3) of every CTA of every kernel of
// the last step executed; mq_debug_timeline copies the table out.
#ifdef MQ_TIMELINE
constexpr int TL_KERNELS = 160, TL_CTAS = 148;
__device__ unsigned long long g_tl[TL_KERNELS * TL_CTAS * 8];
#define TL(a, w)                                                                              \
    do {                                                                                      \
        const int cta_ = blockIdx.x;                                                          \
        if (threadIdx.x == 0 && cta_ < TL_CTAS && (unsigned)(a).kseq < (unsigned)TL_KERNELS) {                    \
            unsigned long long t_;                                                            \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                            \
            g_tl[((a).kseq * TL_CTAS + cta_) * 8 + (w)] = t_;                                 \
            if ((w) == 0) {                                                                   \
                unsigned sm_;                                                                 \
                asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_));                              \
                g_tl[((a).kseq * TL_CTAS + cta_) * 8 + 7] = sm_;                              \
            }                                                                                 \
        }                                                                                     \
    } while (0)
#define TL_SYNC() __syncthreads()
#else
#define TL(a, w) do { } while (0)
#define TL_SYNC() do { } while (0)
#endif

struct DecodeArgs {
    const bf16* embed;
    const bf16* final_norm;
    const bf16* lm_head;
    const bf16* cos;
    const bf16* sin;
    bf16* k_cache;
    bf16* v_cache;
    bf16* hidden;
    bf16* qkv;
    bf16* attn;
    bf16* act;
    float* partials;
    unsigned int* counters;
    unsigned long long* slot;
    unsigned int* status;
    const int* in_token;
    int* out_token;
    const int* pos;
    float* logits;
    int vocab;
    int max_seq;
    int nsplit;
    int chunk_cap;
    uint8_t* k8;     // FP8 shadow cache (k_attn_fp8 only): e4m3 [num_layers, 8, max_seq, 128]
    uint8_t* v8;
    const float* k_scale;   // [num_layers, 8]
    const float* v_scale;
    int kseq;        // launch index within the step (timeline builds only)
    int exp_flags;   // experiments (benchmarks only): 1 skip dot products, 2 skip RMSNorm, 4 no weight copies in the per-layer GEMV kernels
};

constexpr int GEMV_THREADS = 256;
constexpr int DOWN_THREADS = 256;
constexpr int MIN_GRID = 128;                 // at most 32 qkv, 24 gate/up and 8 o/down rows per CTA

__device__ __forceinline__ void row_range(int total, int& r0, int& n) {
    r0 = (int)(((long long)blockIdx.x * total) / gridDim.x);
    const int r1 = (int)(((long long)(blockIdx.x + 1) * total) / gridDim.x);
    n = r1 - r0;
}

// ---------------------------------------------------------------- k_qkv
// qkv[r] = bf16( [Wq;Wk;Wv][r,:] . rmsnorm(hidden) ), r in this CTA's rows.
// For layer 0 the residual stream is first gathered from the embedding table.
//
// All four GEMV kernels have the same shape.  Before the dependency wait, warp 0 copies
// the CTA's weight rows (and the norm weight) into shared memory, one bulk copy per row
// so that rows can be padded (mq_device.cuh, mma_gemv).  After the wait the CTA reads the
// activation vector ONCE (every warp of every CTA reading the same sixteen L2 lines
// serialises on those lines for over a microsecond), normalises it cooperatively, and the
// warps split the K dimension of an mma.sync GEMV; partial sums meet in shared memory and
// are added in a fixed order.
constexpr int WPAD = 8;
constexpr int H_LD = H + WPAD, O_LD = QSZ + WPAD, DN_LD = I + WPAD;

// Cooperative RMSNorm of a 1024-wide vector by 256 threads, four elements each:
// xs <- bf16(w * bf16(x * rsqrt(mean(x^2) + eps))).  Two block barriers, the second by the caller.
__device__ __forceinline__ void stage_norm_1024(const DecodeArgs& a, bf16* xs, float* ssp, const uint2 u, const bf16* nrm,
                                                uint64_t* bar, int tid) {
    const float x0 = bf_lo(u.x), x1 = bf_hi(u.x), x2 = bf_lo(u.y), x3 = bf_hi(u.y);
    const float part = warp_sum(fmaf(x0, x0, fmaf(x1, x1, fmaf(x2, x2, x3 * x3))));
    if ((tid & 31) == 0) ssp[tid >> 5] = part;
    __syncthreads();
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < GEMV_THREADS / 32; ++i) ss += ssp[i];
    const float r = 1.0f / sqrtf(ss * (1.0f / H) + RMS_EPS);
    if (!(EXPF(a) & 4)) mbar_wait(bar, 0, a.status);   // norm weight and weight rows have landed
    uint2 o = u;
    if (!(EXPF(a) & 6)) {
        const uint2 wv = *reinterpret_cast<const uint2*>(nrm + tid * 4);
        o.x = pack_bf16x2(rbf(bf_lo(wv.x) * rbf(x0 * r)), rbf(bf_hi(wv.x) * rbf(x1 * r)));
        o.y = pack_bf16x2(rbf(bf_lo(wv.y) * rbf(x2 * r)), rbf(bf_hi(wv.y) * rbf(x3 * r)));
    }
    *reinterpret_cast<uint2*>(xs + tid * 4) = o;
}

__global__ void __launch_bounds__(GEMV_THREADS) k_qkv(DecodeArgs a, MqLayerWeights w, int layer) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* nrm = reinterpret_cast<bf16*>(smem_raw);                // input RMSNorm weight
    bf16* xs = nrm + H;                                           // normalised input vector
    float* red = reinterpret_cast<float*>(xs + H);                // [8 warps][32 rows]
    float* ssp = red + (GEMV_THREADS / 32) * 32;                  // [8]
    uint64_t* bar = reinterpret_cast<uint64_t*>(ssp + 8);
    bf16* wbuf = reinterpret_cast<bf16*>(bar + 2);                // [rows of this CTA][H_LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int r0, n;
    row_range(QKV, r0, n);
    if (warp == 0 && !(EXPF(a) & 4)) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_fence_init();
            mbar_expect_tx(bar, (uint32_t)(n + 1) * H * 2);
            bulk_g2s(nrm, w.input_layernorm, H * 2, bar);
        }
        __syncwarp();
        if (lane < n) {
            const int r = r0 + lane;
            const bf16* src = r < QSZ ? (const bf16*)w.q_proj + (size_t)r * H
                            : r < QSZ + KVSZ ? (const bf16*)w.k_proj + (size_t)(r - QSZ) * H
                                             : (const bf16*)w.v_proj + (size_t)(r - QSZ - KVSZ) * H;
            bulk_g2s(wbuf + (size_t)lane * H_LD, src, H * 2, bar);
        }
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait_cta();
    TL(a, 1);

    const bf16* src = a.hidden;
    if (layer == 0) {
        int tok = ld_cg_i32(a.in_token);
        const int p = ld_cg_i32(a.pos);
        if (blockIdx.x == 0 && tid == 0) {
            if (tok < 0 || tok >= a.vocab) atomicOr(a.status, MQ_STATUS_BAD_TOKEN);
            if (p < 0 || p >= a.max_seq) atomicOr(a.status, MQ_STATUS_BAD_POSITION);
        }
        tok = min(max(tok, 0), a.vocab - 1);
        src = a.embed + (size_t)tok * H;
    }
    const uint2 u = ld_cg_u2(src + tid * 4);
    if (layer == 0 && blockIdx.x == 0) *reinterpret_cast<uint2*>(a.hidden + tid * 4) = u;
    stage_norm_1024(a, xs, ssp, u, nrm, bar, tid);
    __syncthreads();
    TL(a, 2);

    uint32_t rowaddr[2];
#pragma unroll
    for (int t = 0; t < 2; ++t)
        rowaddr[t] = smem_u32(wbuf) + (uint32_t)((min(t * 16 + (lane & 15), n - 1) * H_LD + (lane >> 4) * 8) * 2);
    float c[2][4] = {};
    constexpr int KS = H / 16 / (GEMV_THREADS / 32);   // k-steps per warp
    if (!(EXPF(a) & 1)) mma_gemv<2>(rowaddr, smem_u32(xs), warp * KS, warp * KS + KS, lane, c);
    if ((lane & 3) == 0) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            red[warp * 32 + t * 16 + (lane >> 2)] = c[t][0];
            red[warp * 32 + t * 16 + 8 + (lane >> 2)] = c[t][2];
        }
    }
    __syncthreads();
    if (tid < n) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_THREADS / 32; ++wi) s += red[wi * 32 + tid];
        a.qkv[r0 + tid] = __float2bfloat16_rn(s);
    }
    TL_SYNC();
    TL(a, 3);
}

// ---------------------------------------------------------------- k_attn
// One CTA per (kv head g, split s).  The two query heads 2g and 2g+1 share the
// K/V stream.  The CTA's chunk of cached K and V rows is copied into shared
// memory before the dependency wait (those rows were written by earlier decode
// steps or by prefill); the new position's K/V come from this layer's qkv.
constexpr int ATT_THREADS = 256;
constexpr int ATT_MIN_CHUNK = 64;
constexpr int PART_STRIDE = D + 2;  // m, l, acc[128]

__device__ __forceinline__ void norm_rope_head(const bf16* raw, const bf16* wn, const bf16* cosr, const bf16* sinr,
                                               int lane, float (&lo)[2], float (&hi)[2]) {
    // lane owns elements 2*lane, 2*lane+1 (first half) and 64+2*lane, 64+2*lane+1 (second half)
    const uint32_t ulo = ld_cg_u32(raw + 2 * lane), uhi = ld_cg_u32(raw + 64 + 2 * lane);
    float xl[2] = {bf_lo(ulo), bf_hi(ulo)}, xh[2] = {bf_lo(uhi), bf_hi(uhi)};
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
        // x*cos + rotate_half(x)*sin, rotate_half = (-second half, first half)
        lo[e] = rbf(rbf(nl * clo[e]) + rbf(-nh * slo[e]));
        hi[e] = rbf(rbf(nh * chi[e]) + rbf(nl * shi[e]));
    }
}

// CTAs of the attention grid that have no positions to work on keep their SM's shared-memory
// slot until every working CTA has passed its dependency wait (counters[NKV + 1] counts them,
// the last one publishes the launch's tag in counters[NKV + 2]).  If they left the moment they
// were launched, their SMs could be empty before the next kernel's CTA has arrived, and the
// block scheduler would put two CTAs of that kernel on some of them.  The hold is only a
// scheduling aid: it is bounded and a stale tag merely ends it early.
constexpr long long ATT_HOLD_CYCLES = 200000;
__device__ __forceinline__ void attn_cta_done(const DecodeArgs& a, unsigned int n_working, unsigned int tag) {
    const unsigned int t = atomicAdd(&a.counters[NKV + 1], 1u);
    if (t == n_working - 1u) {
        a.counters[NKV + 1] = 0u;
        __threadfence();
        atomicExch(&a.counters[NKV + 2], tag);
    }
}

constexpr int KV_LD = D + 8;   // K/V rows are padded by 16 bytes in shared memory (conflict-free ldmatrix)

// FP8 = true: the cached rows come from the e4m3 shadow cache (a.k8 / a.v8) and are expanded to f16
// tiles in place; the new position's K / V are quantised with the stored scales, written to both
// caches and attended over in their quantised form; scores carry the K scale, the output the V
// scale (reference: csrc/megakernel/split_decode_gemm.cu:429-493, 950-1310).
template <bool FP8>
__device__ __forceinline__ void attn_body(const DecodeArgs& a, const MqLayerWeights& w, int layer) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int cap = a.chunk_cap;
    bf16* kt = reinterpret_cast<bf16*>(smem_raw);                     // [cap][KV_LD]
    bf16* vt = kt + (size_t)cap * KV_LD;                              // [cap][KV_LD]
    bf16* qs = vt + (size_t)cap * KV_LD;                              // [2][D] normalised, rotated query heads
    bf16* ps = qs + 2 * D;                                            // [8 warps][2][16] probabilities of the warp's tile
    bf16* cst = ps + (ATT_THREADS / 32) * 32;                         // q_norm | k_norm | cos[pos] | sin[pos]
    float* wm = reinterpret_cast<float*>(cst + 4 * D);                // [8][2] per-warp running max
    float* wl = wm + 16;                                              // [8][2] per-warp sum
    float* ml = wl + 16;                                              // [2][2]
    float* wacc = ml + 4;                                             // [8][2][128] per-warp accumulators
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x % NKV, s = blockIdx.x / NKV;   // CTAs beyond 8 * nsplit only hold their SM's slot
    float ks = 1.f, vs = 1.f;                               // FP8: set before the first step, constant afterwards
    if constexpr (FP8) {
        ks = kv_fp8_scale_guard(a.k_scale[layer * NKV + g]);
        vs = kv_fp8_scale_guard(a.v_scale[layer * NKV + g]);
    }
    const int pos = ld_cg_i32(a.pos);
    const bool valid = pos >= 0 && pos < a.max_seq;
    const int len = pos + 1;
    // one CTA per kv head while the context fits its shared memory (no split, no merge);
    // beyond that the positions are spread evenly over the splits
    int chunk = (len + a.nsplit - 1) / a.nsplit;
    chunk = (len <= cap) ? cap : max(ATT_MIN_CHUNK, (chunk + 15) & ~15);
    const int n_act = valid ? (len + chunk - 1) / chunk : 0;
    const bool active = s < a.nsplit && s < n_act && chunk <= cap;
    if (valid && chunk > cap && tid == 0) atomicOr(a.status, MQ_STATUS_BAD_POSITION);
    const int c0 = s * chunk;
    const int n = active ? min(len, c0 + chunk) - c0 : 0;  // positions handled here
    const bool is_last = active && (s == n_act - 1);       // owns the new position
    const int n_cached = is_last ? n - 1 : n;
    const size_t head_off = ((size_t)(layer * NKV + g) * a.max_seq) * D;

    // Everything fetched here was written by earlier steps (or is a weight): 16-byte async
    // copies, issued before the dependency wait, into the padded rows.
    if (active) {
        if (tid < 64) {
            const int v = tid >> 4, c = tid & 15;
            const bf16* src = v == 0 ? (const bf16*)w.q_norm : v == 1 ? (const bf16*)w.k_norm
                            : v == 2 ? a.cos + (size_t)pos * D : a.sin + (size_t)pos * D;
            cp_async16(cst + v * D + c * 8, src + c * 8);
        }
        if constexpr (FP8) {
            // raw e4m3 rows go to the END of each tile array: expanding row r in place (below) then
            // never overwrites a raw row that has not been read (272 r + 256 <= 144 cap + 128 (r + 1))
            const uint8_t* ksrc = a.k8 + head_off + (size_t)c0 * D;
            const uint8_t* vsrc = a.v8 + head_off + (size_t)c0 * D;
            uint8_t* kst = reinterpret_cast<uint8_t*>(kt) + (size_t)cap * (KV_LD * 2 - D);
            uint8_t* vst = reinterpret_cast<uint8_t*>(vt) + (size_t)cap * (KV_LD * 2 - D);
            for (int i = tid; i < n_cached * 8; i += ATT_THREADS) {
                const int r = i >> 3, c = i & 7;
                cp_async16(kst + (size_t)r * D + c * 16, ksrc + (size_t)r * D + c * 16);
                cp_async16(vst + (size_t)r * D + c * 16, vsrc + (size_t)r * D + c * 16);
            }
        } else {
            const bf16* ksrc = a.k_cache + head_off + (size_t)c0 * D;
            const bf16* vsrc = a.v_cache + head_off + (size_t)c0 * D;
            for (int i = tid; i < n_cached * 16; i += ATT_THREADS) {
                const int r = i >> 4, c = i & 15;
                cp_async16(kt + (size_t)r * KV_LD + c * 8, ksrc + (size_t)r * D + c * 8);
                cp_async16(vt + (size_t)r * KV_LD + c * 8, vsrc + (size_t)r * D + c * 8);
            }
        }
        cp_async_commit();
    }
    pdl_trigger();
    pdl_wait_cta();
    TL(a, 1);
    const unsigned int tag = (unsigned int)pos * 64u + (unsigned int)layer + 1u;
    const unsigned int n_working = (unsigned int)(NKV * n_act);
    if (!active) {
        if (tid == 0 && n_act > 0 && chunk <= cap) {
            const long long t0 = clock64();
            unsigned int seen;
            do {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.counters + NKV + 2) : "memory");
            } while (seen != tag && clock64() - t0 < ATT_HOLD_CYCLES);
        }
        return;
    }
    cp_async_wait_all();
    __syncthreads();   // this thread's copies are complete; the barrier makes everybody's visible
    // release the slot holders now: by this time the next kernel's CTA is resident on their SMs
    if (tid == ATT_THREADS - 1) attn_cta_done(a, n_working, tag);
    if constexpr (FP8) {
        // e4m3 -> f16 in place, 64 rows at a time: thread t reads 32 bytes of K and of V of row
        // r0 + t / 4, the block barrier ends all reads of the group, then the padded f16 rows are written
        const uint8_t* kst = reinterpret_cast<const uint8_t*>(kt) + (size_t)cap * (KV_LD * 2 - D);
        const uint8_t* vst = reinterpret_cast<const uint8_t*>(vt) + (size_t)cap * (KV_LD * 2 - D);
        for (int r0 = 0; r0 < n_cached; r0 += 64) {
            const int r = r0 + (tid >> 2), seg = (tid & 3) * 32;
            const bool have = r < n_cached;
            uint4 k0 = make_uint4(0u, 0u, 0u, 0u), k1 = k0, v0 = k0, v1 = k0;
            if (have) {
                k0 = *reinterpret_cast<const uint4*>(kst + (size_t)r * D + seg);
                k1 = *reinterpret_cast<const uint4*>(kst + (size_t)r * D + seg + 16);
                v0 = *reinterpret_cast<const uint4*>(vst + (size_t)r * D + seg);
                v1 = *reinterpret_cast<const uint4*>(vst + (size_t)r * D + seg + 16);
            }
            __syncthreads();
            if (have) {
                uint4* kd = reinterpret_cast<uint4*>(kt + (size_t)r * KV_LD + seg);
                uint4* vd = reinterpret_cast<uint4*>(vt + (size_t)r * KV_LD + seg);
                fp8x16_to_f16x16(k0, kd[0], kd[1]);
                fp8x16_to_f16x16(k1, kd[2], kd[3]);
                fp8x16_to_f16x16(v0, vd[0], vd[1]);
                fp8x16_to_f16x16(v1, vd[2], vd[3]);
            }
        }
    }

    // ---- per-head norm + RoPE of q (both heads), and of the new k; v raw; zero the V rows
    //      between n and the end of the last 16-position tile (they are multiplied by p = 0)
    if (warp < 2) {
        float lo[2], hi[2];
        norm_rope_head(a.qkv + (2 * g + warp) * D, cst, cst + 2 * D, cst + 3 * D, lane, lo, hi);
        *reinterpret_cast<uint32_t*>(qs + warp * D + 2 * lane) = FP8 ? pack_f16x2(lo[0], lo[1]) : pack_bf16x2(lo[0], lo[1]);
        *reinterpret_cast<uint32_t*>(qs + warp * D + 64 + 2 * lane) = FP8 ? pack_f16x2(hi[0], hi[1]) : pack_bf16x2(hi[0], hi[1]);
    } else if (warp == 2 && is_last) {
        float lo[2], hi[2];
        norm_rope_head(a.qkv + QSZ + g * D, cst + D, cst + 2 * D, cst + 3 * D, lane, lo, hi);
        const uint32_t plo = pack_bf16x2(lo[0], lo[1]), phi = pack_bf16x2(hi[0], hi[1]);
        bf16* krow = kt + (size_t)(n - 1) * KV_LD;
        bf16* gk = a.k_cache + head_off + (size_t)pos * D;
        *reinterpret_cast<uint32_t*>(gk + 2 * lane) = plo;
        *reinterpret_cast<uint32_t*>(gk + 64 + 2 * lane) = phi;
        if constexpr (FP8) {
            const float inv = 1.0f / ks;
            const uint32_t qlo = f32x2_to_fp8x2(lo[0] * inv, lo[1] * inv), qhi = f32x2_to_fp8x2(hi[0] * inv, hi[1] * inv);
            uint8_t* g8 = a.k8 + head_off + (size_t)pos * D;
            *reinterpret_cast<uint16_t*>(g8 + 2 * lane) = (uint16_t)qlo;
            *reinterpret_cast<uint16_t*>(g8 + 64 + 2 * lane) = (uint16_t)qhi;
            uint32_t flo, fhi, unused;
            fp8x4_to_f16x4(qlo, flo, unused);
            fp8x4_to_f16x4(qhi, fhi, unused);
            *reinterpret_cast<uint32_t*>(krow + 2 * lane) = flo;
            *reinterpret_cast<uint32_t*>(krow + 64 + 2 * lane) = fhi;
        } else {
            *reinterpret_cast<uint32_t*>(krow + 2 * lane) = plo;
            *reinterpret_cast<uint32_t*>(krow + 64 + 2 * lane) = phi;
        }
    } else if (warp == 3 && is_last) {
        const uint2 u = ld_cg_u2(a.qkv + QSZ + KVSZ + g * D + 4 * lane);
        *reinterpret_cast<uint2*>(a.v_cache + head_off + (size_t)pos * D + 4 * lane) = u;
        if constexpr (FP8) {
            const float inv = 1.0f / vs;
            const uint32_t q4 = f32x4_to_fp8x4(bf_lo(u.x) * inv, bf_hi(u.x) * inv, bf_lo(u.y) * inv, bf_hi(u.y) * inv);
            *reinterpret_cast<uint32_t*>(a.v8 + head_off + (size_t)pos * D + 4 * lane) = q4;
            uint2 f;
            fp8x4_to_f16x4(q4, f.x, f.y);
            *reinterpret_cast<uint2*>(vt + (size_t)(n - 1) * KV_LD + 4 * lane) = f;
        } else {
            *reinterpret_cast<uint2*>(vt + (size_t)(n - 1) * KV_LD + 4 * lane) = u;
        }
    } else if (warp >= 4) {
        const int n16 = (n + 15) & ~15;
        for (int i = (warp - 4) * 32 + lane; i < (n16 - n) * 16; i += 128)
            *reinterpret_cast<uint4*>(vt + (size_t)(n + (i >> 4)) * KV_LD + (i & 15) * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    TL(a, 2);

    // ---- a warp takes 16-position tiles warp, warp + 8, ..: scores = K_tile . q on the tensor
    // cores (positions are the M dimension, the two heads two of the eight N columns), softmax
    // of the tile, probabilities to bf16, out += P . V_tile (heads in M, dims in N).
    {
        const int gi = lane >> 2, ti = lane & 3;
        const float scale = 0.08838834764831845f * ks;  // 1/sqrt(128) (x the K scale)
        float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
        const uint32_t qaddr = smem_u32(qs) + (uint32_t)((gi & 1) * D + 2 * ti) * 2u;
        bf16* pw = ps + warp * 32;
        for (int tile = warp; tile * 16 < n; tile += ATT_THREADS / 32) {
            const uint32_t rowoff = (uint32_t)(((tile * 16 + (lane & 15)) * KV_LD + (lane >> 4) * 8) * 2);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t af[4];
                ldsm4(af, smem_u32(kt) + rowoff + ks * 32);
                uint32_t b0 = lds32(qaddr + ks * 32), b1 = lds32(qaddr + ks * 32 + 16);
                if (gi >= 2) { b0 = 0u; b1 = 0u; }
                mma16816_sel<FP8>(c, af, b0, b1);
            }
            // lanes with ti == 0 hold head 0 / head 1 of positions gi (c[0], c[1]) and gi + 8 (c[2], c[3])
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
                if constexpr (FP8) {   // rounded to bf16 as on the bf16 path; exact in f16 (8 significant bits, e <= 1)
                    __half* ph = reinterpret_cast<__half*>(pw);
                    ph[gi] = __float2half_rn(rbf(e00)); ph[gi + 8] = __float2half_rn(rbf(e10));
                    ph[16 + gi] = __float2half_rn(rbf(e01)); ph[16 + gi + 8] = __float2half_rn(rbf(e11));
                } else {
                    pw[gi] = __float2bfloat16_rn(e00); pw[gi + 8] = __float2bfloat16_rn(e10);
                    pw[16 + gi] = __float2bfloat16_rn(e01); pw[16 + gi + 8] = __float2bfloat16_rn(e11);
                }
            }
            __syncwarp();
            // A = P: row gi is head gi (rows 2..15 are zero)
            uint32_t pa[4] = {0u, 0u, 0u, 0u};
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
                mma16816_sel<FP8>(o[2 * j], pa, bv[0], bv[1]);
                mma16816_sel<FP8>(o[2 * j + 1], pa, bv[2], bv[3]);
            }
            __syncwarp();
        }
        if (lane == 0) { wm[warp * 2] = m0; wm[warp * 2 + 1] = m1; wl[warp * 2] = l0; wl[warp * 2 + 1] = l1; }
        if (gi < 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                *reinterpret_cast<float2*>(wacc + (warp * 2 + gi) * D + j * 8 + 2 * ti) = make_float2(o[j][0], o[j][1]);
        }
    }
    __syncthreads();
    const int hh = tid >> 7, d = tid & 127;
    float acc = 0.f;
    {
        float M = -1e30f;
#pragma unroll
        for (int w8 = 0; w8 < ATT_THREADS / 32; ++w8) M = fmaxf(M, wm[w8 * 2 + hh]);
        float lsum = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < ATT_THREADS / 32; ++w8) {
            const float f = expf(wm[w8 * 2 + hh] - M);
            lsum = fmaf(wl[w8 * 2 + hh], f, lsum);
            acc = fmaf(wacc[(w8 * 2 + hh) * D + d], f, acc);
        }
        if (d == 0) { ml[hh * 2] = M; ml[hh * 2 + 1] = lsum; }
        // every thread of a head needs (M, l): publish through shared memory
        __syncthreads();
        acc *= vs;                          // 1 on the bf16 path
    }
    const int qhead = 2 * g + hh;
    if (n_act == 1) {
        a.attn[qhead * D + d] = __float2bfloat16_rn(acc / ml[hh * 2 + 1]);
        TL_SYNC();
        TL(a, 3);
        return;
    }
    // ---- split-KV: publish the partial, the last CTA of this kv head merges
    float* part = a.partials + ((size_t)qhead * a.nsplit + s) * PART_STRIDE;
    part[2 + d] = acc;
    if (d == 0) { part[0] = ml[hh * 2]; part[1] = ml[hh * 2 + 1]; }
    // the block barrier orders every thread's partial before thread 0's release; the CTA that
    // takes the last ticket acquires the others' partials with the same instruction
    __syncthreads();
    if (tid == 0) {
        unsigned int t;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(t) : "l"(a.counters + g) : "memory");
        s_last = (t == (unsigned int)(n_act - 1));
    }
    __syncthreads();
    TL(a, 3);
    if (!s_last) return;
    // Merge of the n_act (<= 64) partials of this thread's head.  The first sixteen
    // accumulator columns and the (m, l) pairs (split lane and lane + 32 per lane) are
    // requested together, so a merge of up to sixteen splits costs one L2 round trip.
    const int lane_m = tid & 31;
    const float* pbase = a.partials + (size_t)qhead * a.nsplit * PART_STRIDE;
    float v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = (e < n_act) ? ld_cg_f32(pbase + (size_t)e * PART_STRIDE + 2 + d) : 0.f;
    float mj[2] = {-INFINITY, -INFINITY}, lj[2] = {0.f, 0.f};
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int j = lane_m + 32 * h2;
        if (j < n_act) {
            mj[h2] = ld_cg_f32(pbase + (size_t)j * PART_STRIDE);
            lj[h2] = ld_cg_f32(pbase + (size_t)j * PART_STRIDE + 1);
        }
    }
    const float M = warp_max(fmaxf(mj[0], mj[1]));
    float fj[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) fj[h2] = (lane_m + 32 * h2 < n_act) ? expf(mj[h2] - M) : 0.f;
    const float den = warp_sum(lj[0] * fj[0] + lj[1] * fj[1]);
    float num = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) num = fmaf(v[e], __shfl_sync(0xffffffffu, fj[0], e), num);
    for (int j0 = 16; j0 < n_act; j0 += 16) {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = (j0 + e < n_act) ? ld_cg_f32(pbase + (size_t)(j0 + e) * PART_STRIDE + 2 + d) : 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const int j = j0 + e;
            const float f0 = __shfl_sync(0xffffffffu, fj[0], j & 31), f1 = __shfl_sync(0xffffffffu, fj[1], j & 31);
            num = fmaf(v[e], (j < 32) ? f0 : f1, num);
        }
    }
    a.attn[qhead * D + d] = __float2bfloat16_rn(num / den);
    if (tid == 0) a.counters[g] = 0u;
    TL_SYNC();
    TL(a, 3);
}

__global__ void __launch_bounds__(ATT_THREADS) k_attn(DecodeArgs a, MqLayerWeights w, int layer) { attn_body<false>(a, w, layer); }
__global__ void __launch_bounds__(ATT_THREADS) k_attn_fp8(DecodeArgs a, MqLayerWeights w, int layer) { attn_body<true>(a, w, layer); }

// ---------------------------------------------------------------- k_oproj
// hidden[r] = bf16( hidden[r] + bf16( Wo[r,:] . attn ) )
__global__ void __launch_bounds__(GEMV_THREADS) k_oproj(DecodeArgs a, MqLayerWeights w) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                 // the CTA's copy of the attention output
    float* red = reinterpret_cast<float*>(xs + QSZ);              // [8 warps][8 rows]
    uint64_t* bar = reinterpret_cast<uint64_t*>(red + (GEMV_THREADS / 32) * 8);
    bf16* wbuf = reinterpret_cast<bf16*>(bar + 2);                // [rows of this CTA][O_LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int r0, n;
    row_range(H, r0, n);
    if (warp == 0 && !(EXPF(a) & 4)) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_fence_init();
            mbar_expect_tx(bar, (uint32_t)n * QSZ * 2);
        }
        __syncwarp();
        if (lane < n) bulk_g2s(wbuf + (size_t)lane * O_LD, (const bf16*)w.o_proj + (size_t)(r0 + lane) * QSZ, QSZ * 2, bar);
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait_cta();
    TL(a, 1);

    *reinterpret_cast<uint4*>(xs + tid * 8) = ld_cg_u4(a.attn + tid * 8);   // 256 threads x 16 B = 2048 bf16
    unsigned short hb = 0;
    if (tid < n) hb = __ldcg(reinterpret_cast<const unsigned short*>(a.hidden + r0 + tid));
    if (!(EXPF(a) & 4)) mbar_wait(bar, 0, a.status);
    __syncthreads();
    TL(a, 2);

    uint32_t rowaddr[1] = {smem_u32(wbuf) + (uint32_t)((min(lane & 15, n - 1) * O_LD + (lane >> 4) * 8) * 2)};
    float c[1][4] = {};
    constexpr int KS = QSZ / 16 / (GEMV_THREADS / 32);
    if (!(EXPF(a) & 1)) mma_gemv<1>(rowaddr, smem_u32(xs), warp * KS, warp * KS + KS, lane, c);
    if ((lane & 3) == 0) red[warp * 8 + (lane >> 2)] = c[0][0];
    TL(a, 4);
    __syncthreads();
    TL(a, 5);
    if (tid < n) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_THREADS / 32; ++wi) s += red[wi * 8 + tid];
        const float hres = __uint_as_float((uint32_t)hb << 16);
        a.hidden[r0 + tid] = __float2bfloat16_rn(hres + rbf(s));
    }
    TL_SYNC();
    TL(a, 3);
}

// ---------------------------------------------------------------- k_gateup
// act[i] = bf16( bf16(silu(bf16(Wg[i,:].x))) * bf16(Wu[i,:].x) ), x = rmsnorm(hidden)
__global__ void __launch_bounds__(GEMV_THREADS) k_gateup(DecodeArgs a, MqLayerWeights w) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* nrm = reinterpret_cast<bf16*>(smem_raw);                // post-attention RMSNorm weight
    bf16* xs = nrm + H;
    float* red = reinterpret_cast<float*>(xs + H);                // [8 warps][48 rows]
    float* ssp = red + (GEMV_THREADS / 32) * 48;
    uint64_t* bar = reinterpret_cast<uint64_t*>(ssp + 8);
    bf16* wbuf = reinterpret_cast<bf16*>(bar + 2);                // [2 x rows of this CTA][H_LD]: gate rows, then up rows
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int r0, n;
    row_range(I, r0, n);
    if (warp == 0 && !(EXPF(a) & 4)) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_fence_init();
            mbar_expect_tx(bar, (uint32_t)(2 * n + 1) * H * 2);
            bulk_g2s(nrm, w.post_attn_layernorm, H * 2, bar);
        }
        __syncwarp();
        for (int cidx = lane; cidx < 2 * n; cidx += 32) {
            const bf16* src = cidx < n ? (const bf16*)w.gate_proj + (size_t)(r0 + cidx) * H
                                       : (const bf16*)w.up_proj + (size_t)(r0 + cidx - n) * H;
            bulk_g2s(wbuf + (size_t)cidx * H_LD, src, H * 2, bar);
        }
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait_cta();
    TL(a, 1);

    const uint2 u = ld_cg_u2(a.hidden + tid * 4);
    stage_norm_1024(a, xs, ssp, u, nrm, bar, tid);
    __syncthreads();
    TL(a, 2);

    uint32_t rowaddr[3];
#pragma unroll
    for (int t = 0; t < 3; ++t)
        rowaddr[t] = smem_u32(wbuf) + (uint32_t)((min(t * 16 + (lane & 15), 2 * n - 1) * H_LD + (lane >> 4) * 8) * 2);
    float c[3][4] = {};
    constexpr int KS = H / 16 / (GEMV_THREADS / 32);
    if (!(EXPF(a) & 1)) mma_gemv<3>(rowaddr, smem_u32(xs), warp * KS, warp * KS + KS, lane, c);
    if ((lane & 3) == 0) {
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            red[warp * 48 + t * 16 + (lane >> 2)] = c[t][0];
            red[warp * 48 + t * 16 + 8 + (lane >> 2)] = c[t][2];
        }
    }
    __syncthreads();
    if (tid < n) {
        float gsum = 0.f, usum = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_THREADS / 32; ++wi) { gsum += red[wi * 48 + tid]; usum += red[wi * 48 + n + tid]; }
        const float act = rbf(silu_f32(rbf(gsum)));
        a.act[r0 + tid] = __float2bfloat16_rn(act * rbf(usum));
    }
    TL_SYNC();
    TL(a, 3);
}

// ---------------------------------------------------------------- k_down
// hidden[r] = bf16( hidden[r] + bf16( Wd[r,:] . act ) )
__global__ void __launch_bounds__(DOWN_THREADS) k_down(DecodeArgs a, MqLayerWeights w) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                 // the CTA's copy of the MLP activation
    float* red = reinterpret_cast<float*>(xs + I);                // [8 warps][8 rows]
    uint64_t* bar = reinterpret_cast<uint64_t*>(red + (DOWN_THREADS / 32) * 8);
    bf16* wbuf = reinterpret_cast<bf16*>(bar + 2);                // [rows of this CTA][DN_LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int r0, n;
    row_range(H, r0, n);
    if (warp == 0 && !(EXPF(a) & 4)) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_fence_init();
            mbar_expect_tx(bar, (uint32_t)n * I * 2);
        }
        __syncwarp();
        if (lane < n) bulk_g2s(wbuf + (size_t)lane * DN_LD, (const bf16*)w.down_proj + (size_t)(r0 + lane) * I, I * 2, bar);
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait_cta();
    TL(a, 1);

    for (int i = tid; i < I / 8; i += DOWN_THREADS) *reinterpret_cast<uint4*>(xs + i * 8) = ld_cg_u4(a.act + i * 8);
    unsigned short hb = 0;
    if (tid < n) hb = __ldcg(reinterpret_cast<const unsigned short*>(a.hidden + r0 + tid));
    if (!(EXPF(a) & 4)) mbar_wait(bar, 0, a.status);
    __syncthreads();
    TL(a, 2);

    uint32_t rowaddr[1] = {smem_u32(wbuf) + (uint32_t)((min(lane & 15, n - 1) * DN_LD + (lane >> 4) * 8) * 2)};
    float c[1][4] = {};
    constexpr int KS = I / 16 / (DOWN_THREADS / 32);
    if (!(EXPF(a) & 1)) mma_gemv<1>(rowaddr, smem_u32(xs), warp * KS, warp * KS + KS, lane, c);
    if ((lane & 3) == 0) red[warp * 8 + (lane >> 2)] = c[0][0];
    TL(a, 4);
    __syncthreads();
    TL(a, 5);
    if (tid < n) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < DOWN_THREADS / 32; ++wi) s += red[wi * 8 + tid];
        const float hres = __uint_as_float((uint32_t)hb << 16);
        a.hidden[r0 + tid] = __float2bfloat16_rn(hres + rbf(s));
    }
    TL_SYNC();
    TL(a, 3);
}

// ---------------------------------------------------------------- k_lmhead
// logits[r] = bf16( E[r,:] . rmsnorm(hidden) ); token = lowest index of the maximum.
// The 311 MB embedding matrix streams through a 4-stage shared-memory ring fed
// by one producer thread; eight consumer warps take two rows each per stage.
constexpr int LM_ROWS = 16;
constexpr int LM_STAGES = 4;
constexpr int LM_CONSUMERS = 8;
constexpr int LM_THREADS = (LM_CONSUMERS + 1) * 32;

__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

__global__ void __launch_bounds__(LM_THREADS) k_lmhead(DecodeArgs a) {
    TL(a, 0);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    bf16* ring = reinterpret_cast<bf16*>(smem_raw);  // [LM_STAGES][LM_ROWS][H]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)LM_STAGES * LM_ROWS * H * 2);
    uint64_t* empty = full + LM_STAGES;
    unsigned long long* wbest = reinterpret_cast<unsigned long long*>(empty + LM_STAGES);  // [LM_CONSUMERS]
    uint64_t* nbar = reinterpret_cast<uint64_t*>(wbest + LM_CONSUMERS);
    bf16* nrm = reinterpret_cast<bf16*>(nbar + 2);                     // final RMSNorm weight
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = (int)(((long long)blockIdx.x * a.vocab) / gridDim.x);
    const int r1 = (int)(((long long)(blockIdx.x + 1) * a.vocab) / gridDim.x);
    const int n = r1 - r0;
    const int nst = (n + LM_ROWS - 1) / LM_ROWS;

    auto issue = [&](int it) {
        const int s = it % LM_STAGES;
        const int rows = min(LM_ROWS, n - it * LM_ROWS);
        const uint32_t bytes = (uint32_t)rows * H * 2;
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(ring + (size_t)s * LM_ROWS * H, a.lm_head + (size_t)(r0 + it * LM_ROWS) * H, bytes, &full[s]);
    };
    if (tid == LM_CONSUMERS * 32) {
        for (int s = 0; s < LM_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], LM_CONSUMERS); }
        mbar_init(nbar, 1);
        mbar_fence_init();
        mbar_expect_tx(nbar, H * 2);
        bulk_g2s(nrm, a.final_norm, H * 2, nbar);
        for (int it = 0; it < min(nst, LM_STAGES); ++it) issue(it);
    }
    __syncthreads();
    // The trigger comes AFTER the wait: the next decode step may only begin once
    // every kernel of this step has completed, which makes the KV rows written by
    // this step safe to prefetch in the next step's attention prologues.
    pdl_wait_cta();
    TL(a, 1);
    pdl_trigger();

    if (warp == LM_CONSUMERS) {
        if (lane == 0) {
            for (int it = LM_STAGES; it < nst; ++it) {
                const int s = it % LM_STAGES;
                mbar_wait(&empty[s], (uint32_t)((it / LM_STAGES) - 1) & 1u, a.status);
                issue(it);
            }
        }
    } else {
        float x[32];
        load_x_slice(x, a.hidden, lane);
        mbar_wait(nbar, 0, a.status);
        rmsnorm_slice(x, nrm, lane);
        float bestv = -INFINITY;
        int besti = 0x7fffffff;
        for (int it = 0; it < nst; ++it) {
            const int s = it % LM_STAGES;
            const int rows = min(LM_ROWS, n - it * LM_ROWS);
            mbar_wait(&full[s], (uint32_t)(it / LM_STAGES) & 1u, a.status);
            const bf16* st = ring + (size_t)s * LM_ROWS * H;
            const int ra = warp, rb = warp + LM_CONSUMERS;
            float d0 = 0.f, d1 = 0.f;
            if (ra < rows) d0 = dot_slice(st + (size_t)ra * H, x, lane);
            if (rb < rows) d1 = dot_slice(st + (size_t)rb * H, x, lane);
            d0 = rbf(warp_sum(d0));
            d1 = rbf(warp_sum(d1));
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                const int ga = r0 + it * LM_ROWS + ra, gb = r0 + it * LM_ROWS + rb;
                if (ra < rows) {
                    if (a.logits) a.logits[ga] = d0;
                    if (d0 > bestv) { bestv = d0; besti = ga; }
                }
                if (rb < rows) {
                    if (a.logits) a.logits[gb] = d1;
                    if (d1 > bestv) { bestv = d1; besti = gb; }
                }
            }
        }
        if (lane == 0) wbest[warp] = (besti == 0x7fffffff) ? 0ull : argmax_key(bestv, besti);
    }
    __syncthreads();
    if (tid == 0) {
        unsigned long long k = 0ull;
        for (int i = 0; i < LM_CONSUMERS; ++i) k = wbest[i] > k ? wbest[i] : k;
        atomicMax(a.slot, k);
        __threadfence();
        const unsigned int t = atomicAdd(&a.counters[NKV], 1u);
        if (t == gridDim.x - 1) {
            __threadfence();
            const unsigned long long best = atomicExch(a.slot, 0ull);
            *a.out_token = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
            a.counters[NKV] = 0u;
        }
    }
    TL(a, 3);
}

// ---------------------------------------------------------------- small helpers
__global__ void k_fill_iota(int* dst, int start, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = start + i;
}

__global__ void k_find_first_eos(const int* tokens, int n, const int* eos, int n_eos, int* out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    for (int j = 0; j < n_eos; ++j)
        if (t == eos[j]) { atomicMin(out, i); return; }
}

// ---------------------------------------------------------------- host side
struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
};
static DeviceState g_dev[64];

static int rows_per_cta(int total, int grid) { return (total + grid - 1) / grid; }
static size_t smem_qkv(int G) { return 2 * H * 2 + (GEMV_THREADS / 32) * 32 * 4 + 8 * 4 + 16 + (size_t)rows_per_cta(QKV, G) * H_LD * 2; }
static size_t smem_oproj(int G) { return QSZ * 2 + (GEMV_THREADS / 32) * 8 * 4 + 16 + (size_t)rows_per_cta(H, G) * O_LD * 2; }
static size_t smem_gateup(int G) { return 2 * H * 2 + (GEMV_THREADS / 32) * 48 * 4 + 8 * 4 + 16 + (size_t)2 * rows_per_cta(I, G) * H_LD * 2; }
static size_t smem_down(int G) { return I * 2 + (DOWN_THREADS / 32) * 8 * 4 + 16 + (size_t)rows_per_cta(H, G) * DN_LD * 2; }
static size_t smem_lmhead() { return (size_t)LM_STAGES * LM_ROWS * H * 2 + 2 * LM_STAGES * 8 + LM_CONSUMERS * 8 + 16 + H * 2; }
static size_t smem_attn(int cap) { return (size_t)cap * KV_LD * 2 * 2 + (2 * D + (ATT_THREADS / 32) * 32 + 4 * D) * 2 + (16 + 16 + 4) * 4 + 16 * D * 4; }

// Shared-memory slots.  The block scheduler places a CTA wherever its resources fit, and on
// an idle GPU it hands a 148-CTA grid out per GPC, which puts two CTAs on eight SMs and none
// on eight others; with kernels of unequal footprint it packs up to three CTAs of a small
// kernel onto one SM.  A doubled-up SM takes twice as long, and the slowest SM sets the pace
// of every kernel of the chain.  So the kernels of a step ask for shared memory in two
// alternating sizes, A then B then A ..: A + B fill an SM exactly, two A never fit, and in
// the steady state an SM always holds the running kernel's CTA plus the next kernel's
// (which is prefetching its weights), so the slot a finishing CTA leaves takes exactly one
// CTA of the kernel two places later.  Every kernel gets one CTA per SM.
// (1.5 KB of an SM's 228 KB stay free for the 1 KB the system reserves per CTA and for static shared memory.)
constexpr size_t SLOT_A_BYTES = 130 * 1024 + 512, SLOT_B_BYTES = 94 * 1024;
static size_t slot(int index, size_t need) {
    const size_t sz = (index & 1) ? SLOT_B_BYTES : SLOT_A_BYTES;
    return need > sz ? need : sz;
}

constexpr int ATT_MAX_CAP = 384;    // positions per CTA: 384 * 520 B + 3 KB of shared memory
constexpr int ATT_MAX_SPLIT = 64;

constexpr int ATT_ONE_WAVE_SPLIT = 18;   // 8 kv heads x 18 splits = 144 CTAs: the attention grid still fits one CTA per SM
constexpr int ATT_ONE_WAVE_CAP = 144;    // positions per CTA whose K/V rows fit the smaller shared-memory slot
static int attn_nsplit(int max_seq) {
    int ns = (max_seq + 127) / 128;
    if (ns < 1) ns = 1;
    // a cache slightly longer than 18 x 128 positions keeps 18 splits with longer chunks rather
    // than a grid of more CTAs than SMs
    if (ns > ATT_ONE_WAVE_SPLIT && (((max_seq + ATT_ONE_WAVE_SPLIT - 1) / ATT_ONE_WAVE_SPLIT + 15) & ~15) <= ATT_ONE_WAVE_CAP)
        ns = ATT_ONE_WAVE_SPLIT;
    if (ns > ATT_MAX_SPLIT) ns = ATT_MAX_SPLIT;
    return ns;
}
static int attn_cap(int max_seq) {
    const int ns = attn_nsplit(max_seq);
    int cap = ((max_seq + ns - 1) / ns + 15) & ~15;
    if (cap < ATT_MIN_CHUNK) cap = ATT_MIN_CHUNK;
    return cap;
}

static int ensure_device(DeviceState** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        cudaDeviceProp p;
        e = cudaGetDeviceProperties(&p, dev);
        if (e != cudaSuccess) return (int)e;
        st.sm_count = p.multiProcessorCount;
        st.cc_major = p.major;
        st.cc_minor = p.minor;
        if (p.major != 10 || st.sm_count < MIN_GRID) return MQ_ERR_UNSUPPORTED;
// All kernels of the chain ask for the same (maximum) shared-memory carve-out: kernels
// whose carve-out differs cannot be resident on an SM together, which would serialise
// the programmatic-dependent-launch chain.
#define MQ_SET_SMEM(k, bytes)                                                                   \
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slot(0, bytes)); \
    if (e != cudaSuccess) return (int)e;                                                        \
    e = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared); \
    if (e != cudaSuccess) return (int)e;
        MQ_SET_SMEM(k_qkv, smem_qkv(MIN_GRID));
        MQ_SET_SMEM(k_oproj, smem_oproj(MIN_GRID));
        MQ_SET_SMEM(k_gateup, smem_gateup(MIN_GRID));
        MQ_SET_SMEM(k_down, smem_down(MIN_GRID));
        MQ_SET_SMEM(k_lmhead, smem_lmhead());
        MQ_SET_SMEM(k_attn, smem_attn(ATT_MAX_CAP));
        MQ_SET_SMEM(k_attn_fp8, smem_attn(ATT_MAX_CAP));
#undef MQ_SET_SMEM
        st.ready = true;
    }
    *out = &st;
    return MQ_OK;
}

template <typename... KArgs, typename... Args>
static cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Final RMSNorm + LM head + arg-max on buf->hidden (used by the prefill path).
int launch_lmhead_only(const MqModel* model, const MqDecodeBuffers* buf, int* out_token, float* logits, cudaStream_t stream);

static int g_decode_exp_flags = 0;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mq

using namespace mq;

int mq::launch_lmhead_only(const MqModel* model, const MqDecodeBuffers* buf, int* out_token, float* logits, cudaStream_t stream) {
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != MQ_OK) return rc;
    DecodeArgs a = {};
    a.final_norm = (const bf16*)model->final_norm;
    a.lm_head = (const bf16*)model->lm_head;
    a.hidden = (bf16*)buf->hidden;
    a.counters = buf->counters;
    a.slot = buf->argmax_slot;
    a.status = buf->status;
    a.out_token = out_token;
    a.logits = logits;
    a.vocab = model->vocab_size;
    a.max_seq = model->max_seq_len;
    return (int)launch(k_lmhead, dim3(st->sm_count), dim3(LM_THREADS), smem_lmhead(), stream, false, a);
}

#ifdef MQ_DECODE_EXPERIMENTS
// Benchmark builds only (results become meaningless): 1 skip the dot products, 2 skip the
// RMSNorms, 4 no weight copies.  Not part of the public header.
extern "C" int mq_decode_set_experiment(int flags) {
    g_decode_exp_flags = flags;
    return MQ_OK;
}
#endif

extern "C" int mq_abi_version(void) { return 1; }

extern "C" int mq_device_info(int* sm_count, int* cc_major, int* cc_minor) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) return (int)e;
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    return MQ_OK;
}

extern "C" int mq_init_device(void) {
    DeviceState* st = nullptr;
    return ensure_device(&st);
}

extern "C" int mq_decode_attn_nsplit(int max_seq_len) { return attn_nsplit(max_seq_len); }

extern "C" size_t mq_decode_partials_bytes(int max_seq_len) {
    return (size_t)NQ * attn_nsplit(max_seq_len) * PART_STRIDE * sizeof(float);
}

extern "C" int mq_decode_launch_count(int num_layers) { return 5 * num_layers + 1; }

static int decode_impl(const MqModel* model, const MqDecodeBuffers* buf, const MqKvFp8* kv8, const int* in_token, int* out_token,
                       const int* position, float* logits, int flags, void* stream_v) {
    if (!model || !buf || !in_token || !out_token || !position) return MQ_ERR_BAD_ARG;
    if (kv8 && (!kv8->k_fp8 || !kv8->v_fp8 || !kv8->k_scale || !kv8->v_scale)) return MQ_ERR_BAD_ARG;
    if (!model->embed || !model->layers || !model->final_norm || !model->lm_head || !model->cos_table || !model->sin_table)
        return MQ_ERR_BAD_ARG;
    if (model->num_layers <= 0 || model->vocab_size <= 0 || model->max_seq_len <= 0) return MQ_ERR_BAD_ARG;
    if (!buf->k_cache || !buf->v_cache || !buf->hidden || !buf->qkv || !buf->attn_out || !buf->mlp_act || !buf->attn_partials ||
        !buf->counters || !buf->argmax_slot || !buf->status)
        return MQ_ERR_BAD_ARG;
    const int cap = attn_cap(model->max_seq_len);
    const int nsplit = attn_nsplit(model->max_seq_len);
    if (buf->attn_nsplit != nsplit) return MQ_ERR_BAD_ARG;
    if (cap > ATT_MAX_CAP) return MQ_ERR_TOO_LONG;
    const void* al[] = {model->embed, model->lm_head, model->final_norm, model->cos_table, model->sin_table, buf->k_cache,
                        buf->v_cache, buf->hidden, buf->qkv, buf->attn_out, buf->mlp_act};
    for (const void* p : al)
        if (!aligned16(p)) return MQ_ERR_ALIGNMENT;
    DeviceState* st = nullptr;
    int rc = ensure_device(&st);
    if (rc != MQ_OK) return rc;

    cudaStream_t stream = (cudaStream_t)stream_v;
    DecodeArgs a;
    a.embed = (const bf16*)model->embed;
    a.final_norm = (const bf16*)model->final_norm;
    a.lm_head = (const bf16*)model->lm_head;
    a.cos = (const bf16*)model->cos_table;
    a.sin = (const bf16*)model->sin_table;
    a.k_cache = (bf16*)buf->k_cache;
    a.v_cache = (bf16*)buf->v_cache;
    a.hidden = (bf16*)buf->hidden;
    a.qkv = (bf16*)buf->qkv;
    a.attn = (bf16*)buf->attn_out;
    a.act = (bf16*)buf->mlp_act;
    a.partials = buf->attn_partials;
    a.counters = buf->counters;
    a.slot = buf->argmax_slot;
    a.status = buf->status;
    a.in_token = in_token;
    a.out_token = out_token;
    a.pos = position;
    a.logits = logits;
    a.vocab = model->vocab_size;
    a.max_seq = model->max_seq_len;
    a.nsplit = nsplit;
    a.chunk_cap = cap;
    a.exp_flags = g_decode_exp_flags;
    a.kseq = 0;
    a.k8 = kv8 ? (uint8_t*)kv8->k_fp8 : nullptr;
    a.v8 = kv8 ? (uint8_t*)kv8->v_fp8 : nullptr;
    a.k_scale = kv8 ? kv8->k_scale : nullptr;
    a.v_scale = kv8 ? kv8->v_scale : nullptr;

    const bool pdl = !(flags & MQ_FLAG_NO_PDL);
    const int G = st->sm_count;
    cudaError_t e;
    for (int l = 0; l < model->num_layers; ++l) {
        const MqLayerWeights& w = model->layers[l];
        const bool first = (l == 0);
        a.kseq = 5 * l;
        e = launch(k_qkv, dim3(G), dim3(GEMV_THREADS), slot(5 * l, smem_qkv(G)), stream, pdl && (!first || (flags & MQ_FLAG_CHAINED)), a, w, l);
        if (e != cudaSuccess) return (int)e;
        a.kseq = 5 * l + 1;
        e = launch(kv8 ? k_attn_fp8 : k_attn, dim3(NKV * nsplit > G ? NKV * nsplit : G), dim3(ATT_THREADS), slot(5 * l + 1, smem_attn(cap)), stream, pdl, a, w, l);
        if (e != cudaSuccess) return (int)e;
        a.kseq = 5 * l + 2;
        e = launch(k_oproj, dim3(G), dim3(GEMV_THREADS), slot(5 * l + 2, smem_oproj(G)), stream, pdl, a, w);
        if (e != cudaSuccess) return (int)e;
        a.kseq = 5 * l + 3;
        e = launch(k_gateup, dim3(G), dim3(GEMV_THREADS), slot(5 * l + 3, smem_gateup(G)), stream, pdl, a, w);
        if (e != cudaSuccess) return (int)e;
        a.kseq = 5 * l + 4;
        e = launch(k_down, dim3(G), dim3(DOWN_THREADS), slot(5 * l + 4, smem_down(G)), stream, pdl, a, w);
        if (e != cudaSuccess) return (int)e;
    }
    a.kseq = 5 * model->num_layers;
    e = launch(k_lmhead, dim3(G), dim3(LM_THREADS), slot(5 * model->num_layers, smem_lmhead()), stream, pdl, a);
    if (e != cudaSuccess) return (int)e;
    return MQ_OK;
}

extern "C" int mq_launch_decode(const MqModel* model, const MqDecodeBuffers* buf, const int* in_token, int* out_token,
                                const int* position, float* logits, int flags, void* stream_v) {
    return decode_impl(model, buf, nullptr, in_token, out_token, position, logits, flags, stream_v);
}

extern "C" int mq_launch_decode_kv8(const MqModel* model, const MqDecodeBuffers* buf, const MqKvFp8* kv8, const int* in_token,
                                    int* out_token, const int* position, float* logits, int flags, void* stream_v) {
    if (!kv8) return MQ_ERR_BAD_ARG;
    return decode_impl(model, buf, kv8, in_token, out_token, position, logits, flags, stream_v);
}

extern "C" int mq_launch_fill_iota(int* dst, int start, int n, void* stream) {
    if (!dst || n < 0) return MQ_ERR_BAD_ARG;
    if (n == 0) return MQ_OK;
    k_fill_iota<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dst, start, n);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_find_first_eos(const int* tokens, int n, const int* eos_ids, int n_eos, int* out_index, void* stream) {
    if (!tokens || !out_index || n < 0 || n_eos < 0 || (n_eos > 0 && !eos_ids)) return MQ_ERR_BAD_ARG;
    if (n == 0 || n_eos == 0) return MQ_OK;
    k_find_first_eos<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(tokens, n, eos_ids, n_eos, out_index);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- decode step without allocations
// Some hosts of this library may not allocate device memory while they serve:
// a runtime that hands each plug-in a fixed arena at start-up, a real-time loop
// in which cudaMalloc's implicit device synchronisation is forbidden, or a
// process whose memory pool is owned by another component.  For them the
// scratch of one decode step (residual stream, q|k|v, attention output, MLP
// activation, split-KV partials, tickets and the arg-max slot) lives in this
// file-scope device array instead of caller-provided buffers.  Every GPU that
// loads the library holds these bytes until the process exits.
constexpr size_t NA_HIDDEN_OFF = 0;                                   // bf16 [1024]
constexpr size_t NA_QKV_OFF = NA_HIDDEN_OFF + (size_t)H * 2;          // bf16 [4096]
constexpr size_t NA_ATTN_OFF = NA_QKV_OFF + (size_t)QKV * 2;          // bf16 [2048]
constexpr size_t NA_ACT_OFF = NA_ATTN_OFF + (size_t)QSZ * 2;          // bf16 [3072]
constexpr size_t NA_PART_OFF = NA_ACT_OFF + (size_t)I * 2;            // fp32 [16 * 64 * 130]
constexpr size_t NA_PART_BYTES = (size_t)NQ * mq::ATT_MAX_SPLIT * mq::PART_STRIDE * 4;
constexpr size_t NA_CNT_OFF = NA_PART_OFF + NA_PART_BYTES;            // u32 [16]
constexpr size_t NA_SLOT_OFF = NA_CNT_OFF + 64;                       // u64 [1]
constexpr size_t NA_BYTES = NA_SLOT_OFF + 64;
static_assert(NA_BYTES <= MQ_NOALLOC_SCRATCH_BYTES, "static scratch too small");
static_assert(NA_QKV_OFF % 16 == 0 && NA_ATTN_OFF % 16 == 0 && NA_ACT_OFF % 16 == 0 && NA_PART_OFF % 16 == 0 &&
              NA_CNT_OFF % 16 == 0 && NA_SLOT_OFF % 16 == 0, "scratch members must stay 16-byte aligned");

static __device__ __align__(256) unsigned char g_noalloc_scratch[MQ_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a
// device address; the address is looked up once per device, with that device
// current, and cached here.
static unsigned char* g_noalloc_ptr[64] = {nullptr};

extern "C" int mq_launch_decode_noalloc(const MqModel* model, void* k_cache, void* v_cache, const int* in_token,
                                        int* out_token, const int* position, float* logits, unsigned int* status,
                                        int flags, void* stream_v) {
    if (!model || !k_cache || !v_cache || !in_token || !out_token || !position || !status) return MQ_ERR_BAD_ARG;
    if (model->max_seq_len <= 0) return MQ_ERR_BAD_ARG;
    if (model->max_seq_len > MQ_NOALLOC_MAX_SEQ_LEN) return MQ_ERR_TOO_LONG;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return MQ_ERR_UNSUPPORTED;
    if (!g_noalloc_ptr[dev]) {
        // first call on this device: resolve the symbol's device address
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return MQ_ERR_UNSUPPORTED;
        g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    unsigned char* base = g_noalloc_ptr[dev];
    cudaStream_t stream = (cudaStream_t)stream_v;
    // The tickets and the arg-max slot must start at zero; everything else is
    // fully rewritten by the step before it is read.
    e = cudaMemsetAsync(base + NA_CNT_OFF, 0, 128, stream);
    if (e != cudaSuccess) return (int)e;
    MqDecodeBuffers buf;
    buf.k_cache = k_cache;
    buf.v_cache = v_cache;
    buf.hidden = base + NA_HIDDEN_OFF;
    buf.qkv = base + NA_QKV_OFF;
    buf.attn_out = base + NA_ATTN_OFF;
    buf.mlp_act = base + NA_ACT_OFF;
    buf.attn_partials = reinterpret_cast<float*>(base + NA_PART_OFF);
    buf.counters = reinterpret_cast<unsigned int*>(base + NA_CNT_OFF);
    buf.argmax_slot = reinterpret_cast<unsigned long long*>(base + NA_SLOT_OFF);
    buf.status = status;
    buf.attn_nsplit = mq::attn_nsplit(model->max_seq_len);
    // The memset above sits between this step and the previous one, so the first
    // kernel must not be launched as a programmatic dependent of an earlier step.
    return mq_launch_decode(model, &buf, in_token, out_token, position, logits, flags & ~MQ_FLAG_CHAINED, stream_v);
}

#ifdef MQ_TIMELINE
// Timeline builds only: copies the stamp table (TL_KERNELS x TL_CTAS x 4 u64) to the host.
extern "C" int mq_debug_timeline(void* host_out, size_t bytes) {
    if (!host_out || bytes > sizeof(mq::g_tl)) return MQ_ERR_BAD_ARG;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemcpyFromSymbol(host_out, mq::g_tl, bytes);
}
#endif
