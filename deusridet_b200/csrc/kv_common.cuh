// kv_common.cuh — shared device helpers for the paged-KV kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/drkv.h"

namespace drkv {

// Pool strides in elements (src/machina/paged_attention.cu:13-18, 36-64).
struct PoolLayout {
    int64_t kv_plane, block_stride, layer_stride;
    int num_kv_heads, page_size, head_dim, max_pages;
    __host__ __device__ static PoolLayout make(int hkv, int page, int d, int max_pages) {
        PoolLayout l;
        l.kv_plane = (int64_t)hkv * page * d;
        l.block_stride = 2 * l.kv_plane;
        l.layer_stride = (int64_t)max_pages * l.block_stride;
        l.num_kv_heads = hkv;
        l.page_size = page;
        l.head_dim = d;
        l.max_pages = max_pages;
        return l;
    }
    // element offset of (layer, page, kv plane, head, slot, 0)
    __host__ __device__ int64_t row(int layer, int page, int kv, int head, int slot) const {
        return (int64_t)layer * layer_stride + (int64_t)page * block_stride + (int64_t)kv * kv_plane +
               ((int64_t)head * page_size + slot) * head_dim;
    }
};

template <typename T>
struct Elem;
template <>
struct Elem<__half> {
    static constexpr int kUmmaFormat = 0;   // tcgen05 kind::f16 operand format: 0 = f16, 1 = bf16
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    }
};
template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kUmmaFormat = 1;
    static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
};

// sin and cos of a non-negative fp32 angle, evaluated in fp64 with explicitly rounded
// operations only (no libm, no contraction the compiler could choose differently) and
// rounded once to fp32.  The same sequence of IEEE operations on a CPU gives the same bits,
// which is what makes the RoPE'd K bytes reproducible: the reference evaluates
// cosf/sinf(pos * freq) in fp32 on the device (src/machina/layer_attention.cu:44-48),
// whose result depends on the math library and on --use_fast_math.
//   k = nearest integer to x * 2/pi;  r = x - k * pi/2 (two-part pi/2);
//   sin r, cos r by Taylor polynomials in r^2 up to r^17 / r^18 (|r| <= pi/4).
__device__ __forceinline__ void sincos_det(float angle, float& s, float& c) {
    const double kTwoOverPi = 0.63661977236758134308;
    const double kMagic = 6755399441055744.0;      // 1.5 * 2^52: adding it rounds to an integer
    const double kPio2Hi = 1.57079632673412561417;  // pi/2 with the low 20 mantissa bits zero
    const double kPio2Lo = 6.07710050650619224932e-11;
    double x = (double)angle;
    double t = __fma_rn(x, kTwoOverPi, kMagic);
    int k = __double2loint(t);
    double kd = __dadd_rn(t, -kMagic);
    double r = __fma_rn(-kd, kPio2Hi, x);
    r = __fma_rn(-kd, kPio2Lo, r);
    double z = __dmul_rn(r, r);
    double ps = 1.0 / 355687428096000.0;                 // 1/17!
    ps = __fma_rn(ps, z, -1.0 / 1307674368000.0);        // -1/15!
    ps = __fma_rn(ps, z, 1.0 / 6227020800.0);            // 1/13!
    ps = __fma_rn(ps, z, -1.0 / 39916800.0);             // -1/11!
    ps = __fma_rn(ps, z, 1.0 / 362880.0);                // 1/9!
    ps = __fma_rn(ps, z, -1.0 / 5040.0);                 // -1/7!
    ps = __fma_rn(ps, z, 1.0 / 120.0);                   // 1/5!
    ps = __fma_rn(ps, z, -1.0 / 6.0);                    // -1/3!
    double sn = __fma_rn(__dmul_rn(r, z), ps, r);
    double pc = -1.0 / 6402373705728000.0;               // -1/18!
    pc = __fma_rn(pc, z, 1.0 / 20922789888000.0);        // 1/16!
    pc = __fma_rn(pc, z, -1.0 / 87178291200.0);          // -1/14!
    pc = __fma_rn(pc, z, 1.0 / 479001600.0);             // 1/12!
    pc = __fma_rn(pc, z, -1.0 / 3628800.0);              // -1/10!
    pc = __fma_rn(pc, z, 1.0 / 40320.0);                 // 1/8!
    pc = __fma_rn(pc, z, -1.0 / 720.0);                  // -1/6!
    pc = __fma_rn(pc, z, 1.0 / 24.0);                    // 1/4!
    pc = __fma_rn(pc, z, -0.5);                          // -1/2!
    double cs = __fma_rn(z, pc, 1.0);
    float fs = __double2float_rn(sn), fc = __double2float_rn(cs);
    switch (k & 3) {
        case 0: s = fs; c = fc; break;
        case 1: s = fc; c = -fs; break;
        case 2: s = -fs; c = -fc; break;
        default: s = -fc; c = fs; break;
    }
}

// Rotate-half RoPE on one pair, the exact operation order shared with the CPU checker:
//   x0' = fma(x0, c, -(x1 * s)),  x1' = fma(x1, c, x0 * s)
// (src/machina/layer_attention.cu:55-58 writes x0*c - x1*s and x1*c + x0*s.)
__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, float& y0, float& y1) {
    y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
    y1 = __fmaf_rn(x1, c, __fmul_rn(x0, s));
}

struct alignas(16) Vec16 {
    uint32_t w[4];
};

__device__ __forceinline__ Vec16 ldg16(const void* p) {
    Vec16 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void stg16(void* p, const Vec16& v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]),
                 "r"(v.w[3])
                 : "memory");
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may start while its
// predecessor in the stream is still running.  pdl_wait() returns once the predecessor has
// completed and its writes are visible; everything that touches memory shared with earlier
// kernels comes after it.  pdl_launch_dependents() lets the successor's CTAs be scheduled
// as soon as this grid leaves room.  Every kernel of the engine waits, so completion stays
// chained in stream order.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
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
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Error word shared by all kernels of one engine: 0 = fine.  A kernel that gives up on a
// bounded wait stores a code here instead of trapping, so the context stays usable.
enum KernelError : int { KERR_NONE = 0, KERR_WAIT_FULL = 1, KERR_WAIT_EMPTY = 2, KERR_BAD_PAGE = 3, KERR_WAIT_PEER = 4 };

}  // namespace drkv
