// Two small fused kernels for the decode step AROUND the FP8Linear layers of a Llama-style block
// (the reference's demo does these with a dozen eager torch kernels per layer, which on B200 cost
// more time than the FP8 GEMVs themselves):
//   rope_kv_store  rotary embedding of Q and K from the fused QKV projection, Q written
//                  head-major for the attention call, K and V written into the static KV cache
//                  at the tokens' positions -- one launch instead of ~16;
//   silu_mul       silu(gate) * up on the fused gate/up projection -- one launch instead of 2-3.
// Both are plain bandwidth-bound elementwise kernels on 16-bit activations.
#include "common.cuh"

namespace tfp8b {

template <typename T> struct pair_of;
template <> struct pair_of<__half> { using type = __half2; };
template <> struct pair_of<__nv_bfloat16> { using type = __nv_bfloat162; };

__device__ __forceinline__ float2 unpack2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 unpack2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ __half2 pack2(float a, float b, __half2) { return __floats2half2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 pack2(float a, float b, __nv_bfloat162) { return __floats2bfloat162_rn(a, b); }

// qkv [B, T, H + 2*KV, hd]; pos int64 [T]; cos / sin f32 [max_seq, hd/2] (rotate-half convention:
// element i pairs with element i + hd/2); q_out [B, H, T, hd]; k_cache / v_cache [B, KV, max_seq, hd].
// One thread handles two neighbouring i (a 32-bit pair) of both halves of one head.
template <typename T>
__global__ void __launch_bounds__(256) rope_kv_kernel(const T* __restrict__ qkv, const long long* __restrict__ pos,
                                                      const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                      T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                      int B, int Tn, int H, int KV, int hd, int max_seq) {
    using P = typename pair_of<T>::type;
    const int half = hd / 2, pairs = half / 2, heads = H + 2 * KV;
    const long long total = static_cast<long long>(B) * Tn * heads * pairs;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int ip = static_cast<int>(idx % pairs);
        const int h = static_cast<int>((idx / pairs) % heads);
        const int t = static_cast<int>((idx / (static_cast<long long>(pairs) * heads)) % Tn);
        const int b = static_cast<int>(idx / (static_cast<long long>(pairs) * heads * Tn));
        const long long p = pos[t];
        const T* src = qkv + ((static_cast<size_t>(b) * Tn + t) * heads + h) * hd;
        const float2 x1 = unpack2(*reinterpret_cast<const P*>(src + 2 * ip));
        const float2 x2 = unpack2(*reinterpret_cast<const P*>(src + half + 2 * ip));
        T* dst;
        float2 o1 = x1, o2 = x2;
        if (h < H + KV) {                                      // Q and K heads are rotated
            const float2 c = *reinterpret_cast<const float2*>(cosv + p * half + 2 * ip);
            const float2 s = *reinterpret_cast<const float2*>(sinv + p * half + 2 * ip);
            o1 = make_float2(x1.x * c.x - x2.x * s.x, x1.y * c.y - x2.y * s.y);
            o2 = make_float2(x2.x * c.x + x1.x * s.x, x2.y * c.y + x1.y * s.y);
        }
        if (h < H) dst = q_out + ((static_cast<size_t>(b) * H + h) * Tn + t) * hd;
        else if (h < H + KV) dst = k_cache + ((static_cast<size_t>(b) * KV + (h - H)) * max_seq + p) * hd;
        else dst = v_cache + ((static_cast<size_t>(b) * KV + (h - H - KV)) * max_seq + p) * hd;
        *reinterpret_cast<P*>(dst + 2 * ip) = pack2(o1.x, o1.y, P());
        *reinterpret_cast<P*>(dst + half + 2 * ip) = pack2(o2.x, o2.y, P());
    }
}

// gu [rows, 2F] -> out [rows, F] = silu(gu[:, :F]) * gu[:, F:]; eight elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F) {
    using P = typename pair_of<T>::type;
    const int vec = F / 8;
    const long long total = rows * vec;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = idx / vec;
        const int c = static_cast<int>(idx % vec) * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
        const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
        uint4 o;
        const P* gp = reinterpret_cast<const P*>(&g);
        const P* up = reinterpret_cast<const P*>(&u);
        P* op = reinterpret_cast<P*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = unpack2(gp[i]), b = unpack2(up[i]);
            op[i] = pack2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y, P());
        }
        *reinterpret_cast<uint4*>(out + r * F + c) = o;
    }
}

static int grid_of(long long work) {
    long long blocks = (work + 255) / 256;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace tfp8b

using namespace tfp8b;

extern "C" int tfp8b_rope_kv_store(const void* qkv, int dtype, const long long* pos, const float* cosv, const float* sinv,
                                   void* q_out, void* k_cache, void* v_cache, int B, int T, int H, int KV, int hd,
                                   int max_seq, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_rope_kv_store: f16 / bf16 only");
    TFP8B_REQUIRE(B >= 0 && T >= 0 && H > 0 && KV > 0 && hd > 0 && hd % 4 == 0 && max_seq > 0, TFP8B_ERR_INVALID,
                  "tfp8b_rope_kv_store: bad shape");
    if (B == 0 || T == 0) return TFP8B_OK;
    TFP8B_REQUIRE(qkv && pos && cosv && sinv && q_out && k_cache && v_cache, TFP8B_ERR_INVALID, "tfp8b_rope_kv_store: null pointer");
    const long long work = static_cast<long long>(B) * T * (H + 2 * KV) * (hd / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        rope_kv_kernel<__half><<<grid_of(work), 256, 0, st>>>(static_cast<const __half*>(qkv), pos, cosv, sinv, static_cast<__half*>(q_out),
                                                             static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), B, T, H, KV, hd, max_seq);
    else
        rope_kv_kernel<__nv_bfloat16><<<grid_of(work), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(qkv), pos, cosv, sinv,
                                                                    static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                                                                    static_cast<__nv_bfloat16*>(v_cache), B, T, H, KV, hd, max_seq);
    TFP8B_LAUNCH_CHECK("tfp8b_rope_kv_store");
    return TFP8B_OK;
}

extern "C" int tfp8b_silu_mul(const void* gate_up, void* out, int dtype, long long rows, int F, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_silu_mul: f16 / bf16 only");
    TFP8B_REQUIRE(rows >= 0 && F > 0 && F % 8 == 0, TFP8B_ERR_INVALID, "tfp8b_silu_mul: need F %% 8 == 0");
    if (rows == 0) return TFP8B_OK;
    TFP8B_REQUIRE(gate_up && out, TFP8B_ERR_INVALID, "tfp8b_silu_mul: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long work = rows * (F / 8);
    if (dtype == TFP8B_F16) silu_mul_kernel<__half><<<grid_of(work), 256, 0, st>>>(static_cast<const __half*>(gate_up), static_cast<__half*>(out), rows, F);
    else silu_mul_kernel<__nv_bfloat16><<<grid_of(work), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, F);
    TFP8B_LAUNCH_CHECK("tfp8b_silu_mul");
    return TFP8B_OK;
}
