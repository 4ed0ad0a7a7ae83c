// Dynamic Tanh, a norm without statistics: y = tanh(alpha * x) * w + b, alpha one number, w and b a number per
// column.  Nothing is summed over a row, so the kernels are element-wise (four neighbouring columns to a thread
// where the width is a multiple of four).
//
// add_dyt: x += mult * (a + f) on the 32-bit residual stream, a and f the outputs of a layer's two branches (either
//   may be absent; each may come as rows of any type or as 32-bit partial sums [parts][N][D] of a product that split
//   K, added here in a fixed order), and in the same pass h = dyt(x) in the type the next products read.  Without a
//   and f it is the plain norm of x; h may be x itself (32-bit, in place).  The sum, tanh and the affine map are 32-bit.
#include "common.cuh"

namespace hos {

__device__ __forceinline__ float4 dyt_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 dyt_load4(const bf16* p) {
    const uint2 u = *(const uint2*)p;
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void dyt_store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void dyt_store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *(uint2*)p = u;
}

template <typename TA, typename TF, typename TH>
__global__ void __launch_bounds__(256)
add_dyt_vec_kernel(const TA* __restrict__ a, int a_parts, const TF* __restrict__ f, int f_parts, long long plane, float mult,
                   float* x, float alpha, const float* __restrict__ w, const float* __restrict__ b, TH* h, long long total,
                   int D) {
    pdl_enter();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    float4 v = dyt_load4(x + i);
    if (a != nullptr || f != nullptr) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a != nullptr)
            for (int p = 0; p < a_parts; ++p) {
                const float4 c = dyt_load4(a + (size_t)p * plane + i);
                s.x += c.x; s.y += c.y; s.z += c.z; s.w += c.w;
            }
        if (f != nullptr)
            for (int p = 0; p < f_parts; ++p) {
                const float4 c = dyt_load4(f + (size_t)p * plane + i);
                s.x += c.x; s.y += c.y; s.z += c.z; s.w += c.w;
            }
        v = make_float4(fmaf(mult, s.x, v.x), fmaf(mult, s.y, v.y), fmaf(mult, s.z, v.z), fmaf(mult, s.w, v.w));
        dyt_store4(x + i, v);
    }
    if (h == nullptr) return;
    const int d = (int)(i % D);
    const float4 wv = dyt_load4(w + d), bv = dyt_load4(b + d);
    dyt_store4(h + i, make_float4(fmaf(tanhf(alpha * v.x), wv.x, bv.x), fmaf(tanhf(alpha * v.y), wv.y, bv.y),
                                  fmaf(tanhf(alpha * v.z), wv.z, bv.z), fmaf(tanhf(alpha * v.w), wv.w, bv.w)));
}

template <typename TA, typename TF, typename TH>
__global__ void __launch_bounds__(256)
add_dyt_kernel(const TA* __restrict__ a, int a_parts, const TF* __restrict__ f, int f_parts, long long plane, float mult,
               float* x, float alpha, const float* __restrict__ w, const float* __restrict__ b, TH* h, long long total, int D) {
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = x[i];
    if (a != nullptr || f != nullptr) {
        float s = 0.f;
        if (a != nullptr)
            for (int p = 0; p < a_parts; ++p) s += to_float(a[(size_t)p * plane + i]);
        if (f != nullptr)
            for (int p = 0; p < f_parts; ++p) s += to_float(f[(size_t)p * plane + i]);
        v = fmaf(mult, s, v);
        x[i] = v;
    }
    if (h == nullptr) return;
    const int d = (int)(i % D);
    h[i] = from_float<TH>(fmaf(tanhf(alpha * v), w[d], b[d]));
}

}  // namespace hos

using namespace hos;

// a, f: [N][D] of their dtypes (a_parts / f_parts > 1: that many float32 planes of partial sums) or null.  x: float32
// [N][D].  h: [N][D] of h_dtype or null; with float32 it may be x itself.  w, b: [D].
extern "C" int hos_add_dyt(const void* a, int a_dtype, int a_parts, const void* f, int f_dtype, int f_parts, float mult,
                           float* x, float alpha, const float* w, const float* b, void* h, int h_dtype, int N, int D,
                           cudaStream_t stream) {
    if (N <= 0 || D <= 0) return 0;
    if ((a_parts > 1 && a_dtype != kF32) || (f_parts > 1 && f_dtype != kF32))
        HOS_REFUSE("add_dyt: partial sums must be float32");
    if (h != nullptr && (w == nullptr || b == nullptr)) HOS_REFUSE("add_dyt: the norm needs its weight and its bias");
    const long long total = (long long)N * D;
    const bool vec = D % 4 == 0 && ((uintptr_t)x | (uintptr_t)a | (uintptr_t)f | (uintptr_t)h | (uintptr_t)w | (uintptr_t)b) % 16 == 0;
    const long long items = vec ? total / 4 : total;
    const unsigned blocks = (unsigned)((items + 255) / 256);
#define HOS_DYT(TA, TF, TH)                                                                                          \
    do {                                                                                                             \
        if (vec)                                                                                                     \
            launch_pdl(add_dyt_vec_kernel<TA, TF, TH>, dim3(blocks), dim3(256), 0, stream, (const TA*)a, a_parts,    \
                       (const TF*)f, f_parts, total, mult, x, alpha, w, b, (TH*)h, total, D);                        \
        else                                                                                                         \
            launch_pdl(add_dyt_kernel<TA, TF, TH>, dim3(blocks), dim3(256), 0, stream, (const TA*)a, a_parts,        \
                       (const TF*)f, f_parts, total, mult, x, alpha, w, b, (TH*)h, total, D);                        \
    } while (0)
#define HOS_DYT_F(TA, TF)                                                                                            \
    do {                                                                                                             \
        if (h != nullptr && h_dtype == kBF16) HOS_DYT(TA, TF, bf16);                                                 \
        else HOS_DYT(TA, TF, float);                                                                                 \
    } while (0)
    const bool ab = a != nullptr && a_dtype == kBF16, fb = f != nullptr && f_dtype == kBF16;
    if (ab && fb) HOS_DYT_F(bf16, bf16);
    else if (ab) HOS_DYT_F(bf16, float);
    else if (fb) HOS_DYT_F(float, bf16);
    else HOS_DYT_F(float, float);
#undef HOS_DYT_F
#undef HOS_DYT
    return check_launch("add_dyt");
}
