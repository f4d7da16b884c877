// W4A16 linear on CUDA cores: the path for fp32 activations (the reference's "reference and oracle
// testing" overloads), for M beyond the tensor-core kernel's 32 rows, and for shapes the tensor-core
// kernel does not take (K not a multiple of 128, unaligned pointers, group sizes other than 128).
//
// Same contracts as the reference's kernels:
//   linear_int4 / splitk_int4_impl   src/ops/linear.cpp:33-305
//   linear_int4_fused                src/ops/linear.cpp:351-478
//   mlp_gate_up_swiglu_int4          src/ops/linear.cpp:501-602
//   linear_int4_naive                src/ops/linear.cpp:681-730  (generic kernel below, any group size)
// One warp owns two weight rows (or a gate row and its up row) and MB activation rows; a lane
// streams 16 bytes (32 weights, all inside one 128-k group) per row per step, forms the fp32 dot of
// the exact integers with the activations, and adds dot * scale, the reference's association
// (src/ops/linear.cpp:239-287).  The K-reduction finishes with warp shuffles.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "w4a16.h"

namespace xb {

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxProj = 4;

struct SimtProj {
    void* y;
    const uint8_t* w;
    const __half* scales;
    const float* bias;
    long long n;
    long long ldy;
    long long pair_begin;
};

struct SimtParams {
    SimtProj proj[kMaxProj];
    int num;
    int swiglu;
    long long pairs;
    long long m;
    long long k;
    long long groups;
    int group_size;
    const void* x;
};

template <typename OutT>
__device__ __forceinline__ void put(void* y, long long idx, float v);
template <>
__device__ __forceinline__ void put<float>(void* y, long long idx, float v) { static_cast<float*>(y)[idx] = v; }
template <>
__device__ __forceinline__ void put<__half>(void* y, long long idx, float v) {
    static_cast<__half*>(y)[idx] = __float2half_rn(v);
}

__device__ __forceinline__ void load_x32(const __half* x, float* out) {
    const uint4* p = reinterpret_cast<const uint4*>(x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(p + i);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            out[i * 8 + j * 2] = f.x;
            out[i * 8 + j * 2 + 1] = f.y;
        }
    }
}
__device__ __forceinline__ void load_x32(const float* x, float* out) {
    const float4* p = reinterpret_cast<const float4*>(x);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = __ldg(p + i);
        out[i * 4] = v.x;
        out[i * 4 + 1] = v.y;
        out[i * 4 + 2] = v.z;
        out[i * 4 + 3] = v.w;
    }
}

// fp32 dot of 32 activations with 32 int4 weights (16 bytes), nibble i of word j <-> k = 8 j + i,
// value = (int32(word) << (28 - 4 i)) >> 28 as in src/ops/linear.cpp:100-110.
__device__ __forceinline__ float dot32(const uint4& wv, const float* x) {
    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int32_t sp = static_cast<int32_t>(w[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int32_t q = static_cast<int32_t>(static_cast<uint32_t>(sp) << (28 - 4 * i)) >> 28;
            dot = fmaf(x[j * 8 + i], static_cast<float>(q), dot);
        }
    }
    return dot;
}

template <typename InT, typename OutT, int MB>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) w4a16_simt_kernel(const SimtParams p) {
    const int lane = threadIdx.x & 31;
    const long long pair = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (pair >= p.pairs) return;
    const long long m0 = static_cast<long long>(blockIdx.y) * MB;

    int pi = 0;
    if (!p.swiglu) {
#pragma unroll
        for (int i = 1; i < kMaxProj; ++i)
            if (i < p.num && pair >= p.proj[i].pair_begin) pi = i;
    }
    const SimtProj& pa = p.proj[pi];
    const long long local = pair - pa.pair_begin;
    const long long row_a = p.swiglu ? local : 2 * local;
    const long long row_b = p.swiglu ? local : 2 * local + 1;
    const SimtProj& pb = p.swiglu ? p.proj[1] : pa;
    const bool has_b = row_b < pb.n;

    const long long row_bytes = p.k / 2;
    const uint8_t* wa = pa.w + row_a * row_bytes;
    const uint8_t* wb = has_b ? pb.w + row_b * row_bytes : nullptr;
    const __half* sa = pa.scales + row_a * p.groups;
    const __half* sb = has_b ? pb.scales + row_b * p.groups : nullptr;
    const InT* x = static_cast<const InT*>(p.x);

    float acc_a[MB], acc_b[MB];
#pragma unroll
    for (int i = 0; i < MB; ++i) acc_a[i] = acc_b[i] = 0.f;

    const long long k_end = p.groups * 128;
    for (long long k0 = static_cast<long long>(lane) * 32; k0 < k_end; k0 += 1024) {
        const long long g = k0 >> 7;
        const uint4 va = __ldg(reinterpret_cast<const uint4*>(wa + (k0 >> 1)));
        uint4 vb = make_uint4(0, 0, 0, 0);
        if (has_b) vb = __ldg(reinterpret_cast<const uint4*>(wb + (k0 >> 1)));
        const float sca = __half2float(sa[g]);
        const float scb = has_b ? __half2float(sb[g]) : 0.f;
#pragma unroll
        for (int mi = 0; mi < MB; ++mi) {
            if (m0 + mi < p.m) {
                float xv[32];
                load_x32(x + (m0 + mi) * p.k + k0, xv);
                acc_a[mi] += dot32(va, xv) * sca;
                if (has_b) acc_b[mi] += dot32(vb, xv) * scb;
            }
        }
    }

#pragma unroll
    for (int mi = 0; mi < MB; ++mi) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            acc_a[mi] += __shfl_xor_sync(0xffffffffu, acc_a[mi], off);
            acc_b[mi] += __shfl_xor_sync(0xffffffffu, acc_b[mi], off);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int mi = 0; mi < MB; ++mi) {
            const long long m = m0 + mi;
            if (m >= p.m) continue;
            if (p.swiglu) {
                const float g = acc_a[mi];
                const float silu = g / (1.0f + expf(-g));
                put<OutT>(pa.y, m * pa.ldy + row_a, silu * acc_b[mi]);
            } else {
                float va = acc_a[mi];
                if (pa.bias) va += pa.bias[row_a];
                put<OutT>(pa.y, m * pa.ldy + row_a, va);
                if (has_b) {
                    float vb = acc_b[mi];
                    if (pa.bias) vb += pa.bias[row_b];
                    put<OutT>(pa.y, m * pa.ldy + row_b, vb);
                }
            }
        }
    }
}

// Any shape, any group size, any alignment: one thread per output, the naive association of
// src/ops/linear.cpp:703-722 (acc += x * (q * scale), k ascending).
template <typename InT, typename OutT>
__global__ void w4a16_generic_kernel(const SimtParams p) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    long long total_n = 0;
    for (int i = 0; i < (p.swiglu ? 1 : p.num); ++i) total_n += p.proj[i].n;
    if (idx >= p.m * total_n) return;
    const long long m = idx / total_n;
    long long n = idx % total_n;
    int pi = 0;
    if (!p.swiglu)
        while (n >= p.proj[pi].n) { n -= p.proj[pi].n; ++pi; }
    const InT* x = static_cast<const InT*>(p.x) + m * p.k;
    const int passes = p.swiglu ? 2 : 1;
    float res[2] = {0.f, 0.f};
    for (int ps = 0; ps < passes; ++ps) {
        const SimtProj& pr = p.proj[p.swiglu ? ps : pi];
        const uint8_t* w = pr.w + n * (p.k / 2);
        const __half* sc = pr.scales + n * p.groups;
        float acc = 0.f;
        for (long long g = 0; g < p.groups; ++g) {
            const float scale = __half2float(sc[g]);
            const long long base = g * p.group_size;
            for (int b = 0; b < p.group_size / 2; ++b) {
                const uint8_t byte = w[base / 2 + b];
                int lo = byte & 0x0F;
                if (lo >= 8) lo -= 16;
                int hi = (byte >> 4) & 0x0F;
                if (hi >= 8) hi -= 16;
                acc += static_cast<float>(x[base + 2 * b]) * (static_cast<float>(lo) * scale);
                acc += static_cast<float>(x[base + 2 * b + 1]) * (static_cast<float>(hi) * scale);
            }
        }
        res[ps] = acc;
    }
    const SimtProj& po = p.proj[p.swiglu ? 0 : pi];
    if (p.swiglu) {
        const float silu = res[0] / (1.0f + expf(-res[0]));
        put<OutT>(po.y, m * po.ldy + n, silu * res[1]);
    } else {
        float v = res[0];
        if (po.bias) v += po.bias[n];
        put<OutT>(po.y, m * po.ldy + n, v);
    }
}

template <typename InT, typename OutT>
cudaError_t launch_typed(cudaStream_t stream, const SimtParams& p, bool fast) {
    if (!fast) {
        long long total_n = 0;
        for (int i = 0; i < (p.swiglu ? 1 : p.num); ++i) total_n += p.proj[i].n;
        const long long total = p.m * total_n;
        const int threads = 128;
        w4a16_generic_kernel<InT, OutT><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(p);
        return cudaGetLastError();
    }
    const unsigned blocks = static_cast<unsigned>((p.pairs + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const int threads = kWarpsPerBlock * 32;
    if (p.m == 1) {
        w4a16_simt_kernel<InT, OutT, 1><<<dim3(blocks, 1), threads, 0, stream>>>(p);
    } else if (p.m == 2) {
        w4a16_simt_kernel<InT, OutT, 2><<<dim3(blocks, 1), threads, 0, stream>>>(p);
    } else {
        const unsigned my = static_cast<unsigned>((p.m + 3) / 4);
        w4a16_simt_kernel<InT, OutT, 4><<<dim3(blocks, my), threads, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace

int simt_launch(cudaStream_t stream, const void* x, ActType in, bool out_f32, const TcProj* proj, int num,
                bool swiglu, long long m, long long k, int group_size) {
    SimtParams p{};
    p.num = swiglu ? 2 : num;
    p.swiglu = swiglu ? 1 : 0;
    p.m = m;
    p.k = k;
    p.group_size = group_size;
    p.groups = k / group_size;
    p.x = x;
    bool fast = (group_size == 128) && (k % 128 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    long long pairs = 0;
    for (int i = 0; i < p.num; ++i) {
        p.proj[i].y = proj[i].y;
        p.proj[i].w = proj[i].w;
        p.proj[i].scales = static_cast<const __half*>(proj[i].scales);
        p.proj[i].bias = proj[i].bias;
        p.proj[i].n = proj[i].n;
        p.proj[i].ldy = proj[i].ldy > 0 ? proj[i].ldy : proj[i].n;
        p.proj[i].pair_begin = pairs;
        if (swiglu) {
            if (i == 0) pairs += proj[0].n;
            else p.proj[i].pair_begin = 0;
        } else {
            pairs += (proj[i].n + 1) / 2;
        }
        if (reinterpret_cast<uintptr_t>(proj[i].w) & 15) fast = false;
    }
    p.pairs = pairs;
    if (p.groups <= 0 || pairs <= 0) return 0;
    cudaError_t e;
    if (in == ActType::F16) {
        e = out_f32 ? launch_typed<__half, float>(stream, p, fast) : launch_typed<__half, __half>(stream, p, fast);
    } else {
        e = out_f32 ? launch_typed<float, float>(stream, p, fast) : launch_typed<float, __half>(stream, p, fast);
    }
    return e == cudaSuccess ? 0 : -1;
}

}  // namespace xb
