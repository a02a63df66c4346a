// HBM-bound row-wise stages of the backward: the delta stage that runs before
// the GEMM kernel and the dQ scale+convert stage that runs after it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "geometry.h"

namespace fa3b200 {

constexpr float kLog2E = 1.44269504088896340736f;

__device__ __forceinline__ uint4 ld_stream_16B(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// delta[r] = sum_d dO[r,d] * O[r,d] in fp32, plus the packed sidecar
// {m, r, delta} (definition: reference src/dot_do_o_kernel.cpp:26-63).  Each
// row is owned by D/8 adjacent lanes that each fetch one 16-byte vector of dO
// and of O, so a warp reads 512 contiguous bytes per tensor per instruction.
// When zero_rows is non-null the same lanes also clear the row of the fp32 dQ
// accumulator (row pitch D floats), which saves a separate memset pass.  The
// sidecar is optional (null: only delta is written).
//
// Rows are numbered in [batch, head, row] order (the order of aux0, delta and
// the sidecar); RowLayout says where row r of dO and O lives, so that both the
// [B,H,S,D] and the [B,S,H,D] layout are read in place.  A row whose softmax
// saw no key at all (aux0 = -inf) gets m = 0, r = 0, which makes P zero.
//
// Algorithmic HBM bytes per row: 2*D*2 (dO, O) + 4 (aux0) [+4 aux1] + 4
// (delta) + 12 (sidecar) [+ 4*D when clearing the accumulator].
struct RowLayout {
    TensorStrides strides;  // element strides of the 16-bit tensor
    int heads;
    int seqlen;
    int contiguous;         // 1: row r starts at element r*D ([B,H,S,D] contiguous)
};

__device__ __forceinline__ int64_t row_offset(const RowLayout& l, int64_t row, int d) {
    if (l.contiguous) return row * d;
    const int64_t bh = row / l.seqlen;
    const int s = int(row - bh * l.seqlen);
    const int64_t b = bh / l.heads;
    const int h = int(bh - b * l.heads);
    return b * l.strides.batch + h * l.strides.head + s * l.strides.row;
}

template <typename T, int D, bool kLseInput>
__global__ void __launch_bounds__(256)
delta_sidecar_kernel(const T* __restrict__ dout, const T* __restrict__ out,
                     const float* __restrict__ aux0, const float* __restrict__ aux1,
                     float* __restrict__ delta, float* __restrict__ sidecar,
                     float* __restrict__ zero_rows, int64_t rows, float scale_log2, RowLayout layout) {
    constexpr int kLanesPerRow = D / 8;
    constexpr int kRowsPerWarp = 32 / kLanesPerRow;
    const int lane = threadIdx.x & 31;
    const int sub = lane / kLanesPerRow;
    const int col = lane % kLanesPerRow;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    // Launched programmatically: when the kernel in front lets its dependents go early (the convert
    // kernel of a preceding call does), the blocks are in place when it ends.  Nothing is read or
    // written before all of it has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // let the GEMM kernel behind this one start its set-up (it waits before it reads our outputs)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef FA3B200_TRACE
    if (threadIdx.x == 0) atomicMin(reinterpret_cast<unsigned long long*>(&g_trace_rowwise[0]), (unsigned long long)trace_globaltimer());
#endif

    // the loop bound is the same for every lane of a warp (the shuffles below need all 32 lanes);
    // lanes whose row lies past the end compute on zeros and write nothing
    for (int64_t base = warp * kRowsPerWarp; base < rows; base += warps * kRowsPerWarp) {
        const int64_t row = base + sub;
        const bool valid = row < rows;
        uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
        if (valid) {
            const int64_t src = row_offset(layout, row, D) + col * 8;
            a = ld_stream_16B(dout + src);
            b = ld_stream_16B(out + src);
        }
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x = unpack2<T>(aw[i]);
            const float2 y = unpack2<T>(bw[i]);
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
        }
#pragma unroll
        for (int off = kLanesPerRow / 2; off > 0; off >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, off);
        }
        if (valid && zero_rows != nullptr) {
            float4* z = reinterpret_cast<float4*>(zero_rows + row * D);
#pragma unroll
            for (int i = 0; i < (D / 4) / kLanesPerRow; ++i) {
                z[col + i * kLanesPerRow] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (valid && col == 0) delta[row] = acc;
        if (valid && col == 0 && sidecar != nullptr) {
            float m, r;
            if (kLseInput) {
                m = aux0[row] * kLog2E;
                r = 1.0f;
            } else {
                m = aux0[row] * scale_log2;
                const float sum = aux1[row];
                r = sum != 0.0f ? 1.0f / sum : 0.0f;
            }
            if (m == -INFINITY) {  // no visible key
                m = 0.0f;
                r = 0.0f;
            }
            float* s = sidecar + row * 3;
            s[0] = m;
            s[1] = r;
            s[2] = acc;
        }
    }
#ifdef FA3B200_TRACE
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned long long*>(&g_trace_rowwise[1]), (unsigned long long)trace_globaltimer());
#endif
}

// Up to three (fp32 -> storage dtype) conversions in one launch: dQ (scaled) from its accumulator
// always; dK and dV as well when key tiles were split.  A split tile's dK / dV is the sum of the
// per-CTA slabs its chunks wrote ([128 rows][D] fp32 each, dK slab then dV slab per CTA), added here
// in chunk order, so these two outputs do not depend on the order in which the CTAs ran.  The slabs
// hold fp16 when the inputs are fp16 and fp32 when they are bf16.
constexpr int kMaxSplitTiles = 148;  // tiles are only split while tiles x heads < 148
struct ConvertSegments {
    const float* src[3];   // [0]: fp32 dQ accumulator [batch, head, row, D] contiguous; [1],[2] unused
    void* dst[3];
    int64_t n_vec8[3];
    float scale[3];
    RowLayout layout[3];   // where the rows of dst live
    int count;
    int head_dim;
    const void* slabs;     // count == 3: slab base; chunk x of the GEMM kernel owns slabs 2x (dK) and 2x+1 (dV)
    int slabs_f16;         // the slabs hold fp16 (fp16 inputs) instead of fp32
    int rows_k;            // key rows per (batch, KV head)
    int chunks_per_head;   // CTAs per (batch, KV head)
    unsigned short chunk_begin[kMaxSplitTiles + 1];  // first chunk of key tile kt inside its head
};

// dst[i] = T(scale * accum[i]).  8 elements per thread: 32 B in, 16 B out.
// Algorithmic HBM bytes per element: 4 read + 2 written.
// kSlabs = false: dQ alone (every problem whose key tiles are not split), a lean single-segment loop.
template <typename T, bool kSlabs>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const __grid_constant__ ConvertSegments seg) {
#ifdef FA3B200_TRACE
    if (threadIdx.x == 0) atomicMin(reinterpret_cast<unsigned long long*>(&g_trace_rowwise[2]), (unsigned long long)trace_globaltimer());
#endif
    // launched programmatically behind the GEMM kernel: wait until all of it has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // (a following call's first kernel may take its place now; it waits for this one itself)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // The segments form one index space, so that with enough blocks every thread makes a single
    // load -> store trip whatever the number of segments (small problems are latency-bound here).
    const int64_t n0 = seg.n_vec8[0];
    const int64_t n01 = n0 + (kSlabs ? seg.n_vec8[1] : 0);
    const int64_t total = n01 + (kSlabs ? seg.n_vec8[2] : 0);
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int vec_per_row = seg.head_dim / 8;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += stride) {
        // (selects instead of indexing: the parameter arrays stay in constant memory)
        const int sgi = !kSlabs ? 0 : (g < n0 ? 0 : (g < n01 ? 1 : 2));
        const int64_t i = g - (sgi == 0 ? 0 : (sgi == 1 ? n0 : n01));
        T* __restrict__ dst = static_cast<T*>(sgi == 0 ? seg.dst[0] : (sgi == 1 ? seg.dst[1] : seg.dst[2]));
        const float scale = sgi == 0 ? seg.scale[0] : (sgi == 1 ? seg.scale[1] : seg.scale[2]);
        float v[8];
        if (sgi == 0) {
            const uint4 lo = ld_stream_16B(seg.src[0] + i * 8);
            const uint4 hi = ld_stream_16B(seg.src[0] + i * 8 + 4);
            v[0] = __uint_as_float(lo.x); v[1] = __uint_as_float(lo.y);
            v[2] = __uint_as_float(lo.z); v[3] = __uint_as_float(lo.w);
            v[4] = __uint_as_float(hi.x); v[5] = __uint_as_float(hi.y);
            v[6] = __uint_as_float(hi.z); v[7] = __uint_as_float(hi.w);
        } else {
            // element (head, row, col) of dK / dV: add the slabs of the chunks of key tile row / 128
            const int64_t row_all = i / vec_per_row;
            const int col = int(i - row_all * vec_per_row) * 8;
            const int64_t bh = row_all / seg.rows_k;
            const int row = int(row_all - bh * seg.rows_k);
            const int kt = row >> 7;
            const int c0 = seg.chunk_begin[kt], c1 = seg.chunk_begin[kt + 1];
            const int64_t slab_elems = int64_t(kTileRows) * seg.head_dim;
            const int64_t first = ((bh * seg.chunks_per_head + c0) * 2 + (sgi - 1)) * slab_elems +
                                  int64_t(row & 127) * seg.head_dim + col;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.0f;
            if (seg.slabs_f16) {
                const __half* src = static_cast<const __half*>(seg.slabs) + first;
                for (int c = c0; c < c1; ++c, src += 2 * slab_elems) {
                    const uint4 x = ld_stream_16B(src);
                    const float2 a0 = unpack2<__half>(x.x), a1 = unpack2<__half>(x.y);
                    const float2 a2 = unpack2<__half>(x.z), a3 = unpack2<__half>(x.w);
                    v[0] += a0.x; v[1] += a0.y; v[2] += a1.x; v[3] += a1.y;
                    v[4] += a2.x; v[5] += a2.y; v[6] += a3.x; v[7] += a3.y;
                }
            } else {
                const float* src = static_cast<const float*>(seg.slabs) + first;
                for (int c = c0; c < c1; ++c, src += 2 * slab_elems) {
                    const uint4 lo = ld_stream_16B(src);
                    const uint4 hi = ld_stream_16B(src + 4);
                    v[0] += __uint_as_float(lo.x); v[1] += __uint_as_float(lo.y);
                    v[2] += __uint_as_float(lo.z); v[3] += __uint_as_float(lo.w);
                    v[4] += __uint_as_float(hi.x); v[5] += __uint_as_float(hi.y);
                    v[6] += __uint_as_float(hi.z); v[7] += __uint_as_float(hi.w);
                }
            }
        }
        uint4 o;
        o.x = pack2<T>(v[0] * scale, v[1] * scale);
        o.y = pack2<T>(v[2] * scale, v[3] * scale);
        o.z = pack2<T>(v[4] * scale, v[5] * scale);
        o.w = pack2<T>(v[6] * scale, v[7] * scale);
        // (the layout of a call is the same for all its segments up to heads and rows)
        const bool contiguous = seg.layout[0].contiguous != 0;
        if (contiguous) {
            reinterpret_cast<uint4*>(dst)[i] = o;
        } else {
            const RowLayout layout = sgi == 0 ? seg.layout[0] : (sgi == 1 ? seg.layout[1] : seg.layout[2]);
            const int64_t row = i / vec_per_row;
            const int col = int(i - row * vec_per_row) * 8;
            *reinterpret_cast<uint4*>(dst + row_offset(layout, row, seg.head_dim) + col) = o;
        }
    }
#ifdef FA3B200_TRACE
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned long long*>(&g_trace_rowwise[3]), (unsigned long long)trace_globaltimer());
#endif
}

}  // namespace fa3b200
