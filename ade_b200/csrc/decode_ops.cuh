// Small fused kernels for the token-by-token decode step of a LLaMA-architecture model.
//
// They are not part of the delta application itself.  At decode sizes a Hugging Face decoder layer runs about forty
// elementwise kernels around the four launches of the factored kernel (RMSNorm: 8 each, rotary embedding: 14, SiLU
// and product: 2), and inside a CUDA graph every one of them costs about as much as it would take to stream a
// megabyte of weights.  The three kernels here do the same arithmetic with the same bfloat16 roundings in one launch
// each, so that tokens/s measures the weight stream and not the launch count.  No counterpart in the reference, which
// leaves these operations to transformers (src/evaluate.py:241 calls model.generate).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ade {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out[t][:] = w * bf16(x[t][:] * rsqrt(mean(x[t][:]^2) + eps)): float32 statistics, the normalised value rounded to
// bfloat16 before the (bfloat16) multiplication by the weight, as LlamaRMSNorm.forward does.  One CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ out, int H, long long x_stride, float eps) {
    __shared__ float part[8];
    const __nv_bfloat16* xr = x + static_cast<size_t>(blockIdx.x) * x_stride;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = __bfloat162float(xr[i]);
        s += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
    __nv_bfloat16* orow = out + static_cast<size_t>(blockIdx.x) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float n = bf16r(__bfloat162float(xr[i]) * inv);
        orow[i] = __float2bfloat16_rn(__bfloat162float(w[i]) * n);
    }
}

// Rotary position embedding of q and k in one launch (apply_rotary_pos_emb of transformers' LLaMA model):
//   out[i] = bf16(bf16(x[i] cos[i]) + bf16(rot[i] sin[i])),  rot = (-x[hd/2:], x[:hd/2]),
// every product and the sum rounded to bfloat16 as the elementwise torch operations round them.
// x is read as [B][T][heads][hd] with a row stride (the projections may be column slices of a fused output); the
// result is written as [B][heads][T][hd], the layout attention and the KV cache take.  cos / sin: [B or 1][T][hd]
// (cs_batch_stride = T * hd, or 0 when one table serves every batch row).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ cs,
                            const __nv_bfloat16* __restrict__ sn, __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko, int B, int T,
                            int hq, int hk, int hd, long long q_stride, long long k_stride, long long cs_batch_stride) {
    const int half = hd >> 1;
    const long long total = static_cast<long long>(B) * T * (hq + hk) * hd;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total; e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % hd);
        long long r = e / hd;
        const int h = static_cast<int>(r % (hq + hk));
        r /= (hq + hk);
        const int t = static_cast<int>(r % T), b = static_cast<int>(r / T);
        const bool is_q = h < hq;
        const int hh = is_q ? h : h - hq;
        const __nv_bfloat16* src = (is_q ? q + (static_cast<long long>(b) * T + t) * q_stride : k + (static_cast<long long>(b) * T + t) * k_stride) + hh * hd;
        const float x = __bfloat162float(src[d]);
        const float other = d < half ? -__bfloat162float(src[d + half]) : __bfloat162float(src[d - half]);
        const size_t ci = static_cast<size_t>(b) * cs_batch_stride + static_cast<size_t>(t) * hd + d;
        const float v = bf16r(bf16r(x * __bfloat162float(cs[ci])) + bf16r(other * __bfloat162float(sn[ci])));
        __nv_bfloat16* dst = is_q ? qo + ((static_cast<size_t>(b) * hq + hh) * T + t) * hd : ko + ((static_cast<size_t>(b) * hk + hh) * T + t) * hd;
        dst[d] = __float2bfloat16_rn(v);
    }
}

// out = bf16(bf16(silu(g)) * u), silu evaluated in float32 as torch evaluates it for a bfloat16 tensor.
// g and u are [rows][cols] with row strides (column slices of a fused gate/up output), out is contiguous.
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ out,
                                int rows, int cols, long long g_stride, long long u_stride) {
    const long long total = static_cast<long long>(rows) * cols;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total; e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = e / cols;
        const int c = static_cast<int>(e - r * cols);
        const float x = __bfloat162float(g[r * g_stride + c]);
        const float s = bf16r(x / (1.0f + expf(-x)));
        out[e] = __float2bfloat16_rn(s * __bfloat162float(u[r * u_stride + c]));
    }
}

}  // namespace ade
