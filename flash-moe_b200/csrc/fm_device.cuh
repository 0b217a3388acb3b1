// Device-side building blocks shared by the kernels: async copies, ldmatrix / mma.sync wrappers,
// bf16 packing, fast exp2, shared-memory swizzle.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fm {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte global -> shared asynchronous copy, bypassing L1 (streamed once).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                            uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// x = hi + lo with hi = bf16(x), lo = bf16(x - hi): two bf16 terms carry ~16 mantissa bits.
__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16 &hi, __nv_bfloat16 &lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}
// Packed pair version: hi = x truncated to bf16 (a byte permute, exact), lo = bf16(x - hi).
// x - hi is exact in fp32, so hi + lo carries 16 mantissa bits whichever way hi was rounded.
__device__ __forceinline__ void split_pack_bf16(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    const uint32_t u0 = __float_as_uint(x0), u1 = __float_as_uint(x1);
    hi = __byte_perm(u0, u1, 0x7632);  // {x1[31:16], x0[31:16]}
    const float r0 = x0 - __uint_as_float(u0 & 0xffff0000u);
    const float r1 = x1 - __uint_as_float(u1 & 0xffff0000u);
    lo = pack_bf16(r0, r1);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm volatile("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 1 / (1 + e^-x) from the two special-function approximations (ex2: 2 ulp, rcp: 1 ulp)
__device__ __forceinline__ float fast_sigmoid(float x) { return fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * x)); }

// sin and cos of an fp32 angle of any size: the angle is brought into [-pi, pi] in double precision
// (three fp64 operations) so that sincosf never takes its large-argument path, which costs
// microseconds at positions beyond ~1e5.  Agrees with libm's sinf / cosf of the same fp32 angle to
// about 1e-7 absolute.
__device__ __forceinline__ void sincos_reduced(float ang, float &sn, float &cs) {
    const double a = (double)ang;
    const double k = rint(a * 0.15915494309189535);  // 1 / (2 pi)
    sincosf((float)(a - k * 6.283185307179586), &sn, &cs);
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
    return __uint_as_float(static_cast<uint32_t>(b) << 16);
}

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

// Rows of 512 B (256 bf16) in shared memory: 16-byte chunk c of row r is stored at chunk
// c ^ (r & 7), so that the eight row addresses of an 8x8 ldmatrix tile hit distinct banks.
__device__ __forceinline__ uint32_t swz_row512(int row, int chunk) {
    return static_cast<uint32_t>(row) * 512u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1.0e30f;  // "minus infinity" that survives subtraction

}  // namespace fm
