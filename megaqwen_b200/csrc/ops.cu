// Standalone bf16 ops with the arithmetic and rounding points of the fused
// kernels, for callers that compose a model op by op.  They replace the
// reference's csrc/kernels extension (rms_norm.cu:60-170, silu_mul.cu:22-111,
// rope.cu:31-188, attention_decode.cu:110-357; launch_* declared in
// csrc/kernels/__init__.py:40-95).  General shapes; not performance critical.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mq_device.cuh"

namespace mq {

// out[r,:] = bf16( w * bf16( x[r,:] * rsqrt(mean(x^2) + eps) ) )
__global__ void __launch_bounds__(256) k_op_rms_norm(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ out,
                                                     int n_cols, float eps) {
    __shared__ float s_red[8];
    const int row = blockIdx.x, tid = threadIdx.x;
    const bf16* xr = x + (size_t)row * n_cols;
    float ss = 0.f;
    for (int c = tid; c < n_cols; c += 256) { const float v = bf2f(xr[c]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_red[i];
    const float r = 1.0f / sqrtf(tot / (float)n_cols + eps);
    for (int c = tid; c < n_cols; c += 256)
        out[(size_t)row * n_cols + c] = __float2bfloat16_rn(bf2f(w[c]) * rbf(bf2f(xr[c]) * r));
}

// out = bf16( bf16(silu(gate)) * up )
__global__ void __launch_bounds__(256) k_op_silu_mul(const bf16* __restrict__ gate, const bf16* __restrict__ up, bf16* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(rbf(silu_f32(bf2f(gate[i]))) * bf2f(up[i]));
}

// split-half rotary embedding in bf16: out = bf16( bf16(x*cos) + bf16(rotate_half(x)*sin) )
// x, out: [rows, n_heads, head_dim]; the position of row r is pos0 + r.
__global__ void __launch_bounds__(128) k_op_rope(const bf16* __restrict__ x, const bf16* __restrict__ cos, const bf16* __restrict__ sin,
                                                 bf16* __restrict__ out, int n_heads, int head_dim, int pos0) {
    const int row = blockIdx.x, head = blockIdx.y, half = head_dim / 2;
    const bf16* xr = x + ((size_t)row * n_heads + head) * head_dim;
    bf16* orow = out + ((size_t)row * n_heads + head) * head_dim;
    const bf16* c = cos + (size_t)(pos0 + row) * head_dim;
    const bf16* s = sin + (size_t)(pos0 + row) * head_dim;
    for (int i = threadIdx.x; i < half; i += 128) {
        const float lo = bf2f(xr[i]), hi = bf2f(xr[i + half]);
        orow[i] = __float2bfloat16_rn(rbf(lo * bf2f(c[i])) + rbf(-hi * bf2f(s[i])));
        orow[i + half] = __float2bfloat16_rn(rbf(hi * bf2f(c[i + half])) + rbf(lo * bf2f(s[i + half])));
    }
}

// Single-query attention over a contiguous cache: q [batch, nq, d], caches
// [batch, nkv, max_seq, d], out [batch, nq, d].  fp32 scores and softmax, the
// probabilities rounded to bf16 before the value product, divided by the fp32 sum.
__global__ void __launch_bounds__(128) k_op_attention_decode(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                                             bf16* __restrict__ out, int cache_len, int nq, int nkv, int d, int max_seq,
                                                             float scale) {
    extern __shared__ float sc[];          // [cache_len] scores, then probabilities
    __shared__ float s_red[4];
    const int b = blockIdx.y, h = blockIdx.x, g = h / (nq / nkv), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bf16* qr = q + ((size_t)b * nq + h) * d;
    const bf16* kb = kc + ((size_t)b * nkv + g) * max_seq * d;
    const bf16* vb = vc + ((size_t)b * nkv + g) * max_seq * d;
    for (int p = warp; p < cache_len; p += 4) {     // one warp per key
        float s = 0.f;
        for (int i = lane; i < d; i += 32) s = fmaf(bf2f(qr[i]), bf2f(kb[(size_t)p * d + i]), s);
        s = warp_sum(s);
        if (lane == 0) sc[p] = s * scale;
    }
    __syncthreads();
    float m = -INFINITY;
    for (int p = tid; p < cache_len; p += 128) m = fmaxf(m, sc[p]);
    m = warp_max(m);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    __syncthreads();
    float l = 0.f;
    for (int p = tid; p < cache_len; p += 128) { const float e = expf(sc[p] - m); l += e; sc[p] = rbf(e); }
    l = warp_sum(l);
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    l = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    for (int i = tid; i < d; i += 128) {
        float acc = 0.f;
        for (int p = 0; p < cache_len; ++p) acc = fmaf(sc[p], bf2f(vb[(size_t)p * d + i]), acc);
        out[((size_t)b * nq + h) * d + i] = __float2bfloat16_rn(acc / l);
    }
}

}  // namespace mq

using namespace mq;

extern "C" int mq_launch_rms_norm(const void* x, const void* weight, void* out, int n_rows, int n_cols, float eps, void* stream) {
    if (!x || !weight || !out || n_rows < 0 || n_cols <= 0) return MQ_ERR_BAD_ARG;
    if (n_rows == 0) return MQ_OK;
    k_op_rms_norm<<<n_rows, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)weight, (bf16*)out, n_cols, eps);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_silu_mul(const void* gate, const void* up, void* out, long long n_elements, void* stream) {
    if (!gate || !up || !out || n_elements < 0) return MQ_ERR_BAD_ARG;
    if (n_elements == 0) return MQ_OK;
    k_op_silu_mul<<<(unsigned)((n_elements + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)gate, (const bf16*)up, (bf16*)out, (size_t)n_elements);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_rope(const void* q, const void* k, const void* cos, const void* sin, void* q_out, void* k_out, int seq_len,
                              int n_q_heads, int n_kv_heads, int head_dim, void* stream) {
    if (!q || !k || !cos || !sin || !q_out || !k_out || seq_len < 0 || n_q_heads <= 0 || n_kv_heads <= 0) return MQ_ERR_BAD_ARG;
    if (head_dim <= 0 || (head_dim & 1)) return MQ_ERR_BAD_ARG;
    if (seq_len == 0) return MQ_OK;
    k_op_rope<<<dim3(seq_len, n_q_heads), 128, 0, (cudaStream_t)stream>>>((const bf16*)q, (const bf16*)cos, (const bf16*)sin, (bf16*)q_out, n_q_heads, head_dim, 0);
    k_op_rope<<<dim3(seq_len, n_kv_heads), 128, 0, (cudaStream_t)stream>>>((const bf16*)k, (const bf16*)cos, (const bf16*)sin, (bf16*)k_out, n_kv_heads, head_dim, 0);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_rope_single(const void* x, const void* cos, const void* sin, void* out, int n_heads, int head_dim, int position,
                                     void* stream) {
    if (!x || !cos || !sin || !out || n_heads <= 0 || head_dim <= 0 || (head_dim & 1) || position < 0) return MQ_ERR_BAD_ARG;
    k_op_rope<<<dim3(1, n_heads), 128, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)cos, (const bf16*)sin, (bf16*)out, n_heads, head_dim, position);
    return (int)cudaGetLastError();
}

extern "C" int mq_launch_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, int batch_size, int cache_len,
                                          int n_q_heads, int n_kv_heads, int head_dim, int max_seq_len, float scale, void* stream) {
    if (!q || !k_cache || !v_cache || !out || batch_size <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) return MQ_ERR_BAD_ARG;
    if (n_q_heads % n_kv_heads != 0) return MQ_ERR_BAD_ARG;
    if (cache_len <= 0 || cache_len > max_seq_len) return MQ_ERR_TOO_LONG;
    const size_t smem = (size_t)cache_len * sizeof(float);
    if (smem > 200 * 1024) return MQ_ERR_TOO_LONG;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k_op_attention_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    k_op_attention_decode<<<dim3(n_q_heads, batch_size), 128, smem, (cudaStream_t)stream>>>(
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, cache_len, n_q_heads, n_kv_heads, head_dim, max_seq_len, scale);
    return (int)cudaGetLastError();
}
