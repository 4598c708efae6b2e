// Timestamp-aligned resampling and N-stream temporal fusion for sm_100a.
//
// One kernel serves both operators.  A CTA owns one batch row b and a tile of 32*W
// target times (W warps).  The source timestamp rows of every stream of b are staged in
// shared memory once per CTA.  Each LANE then searches the bracket of its own target in
// shared memory (a branch-free lower bound, the same number of probes in every lane) and
// computes its weight; the warp walks the 32 targets together, fetching bracket index and
// weight from the owning lane with shuffles, and streams the two source rows with
// VEC-byte accesses per lane (16 B = bf16x8 / fp32x4 when sizes and pointers allow),
// writing straight into the stream's column slice of the output row.
//
// Arithmetic follows the reference's torch CPU path op by op, every result rounded
// separately (no FMA contraction, IEEE divide):
//   robocache/python/robocache/ops_fallback.py:132-150
//     idx = clamp(searchsorted_left(st, t), 1, S-1); l = idx-1; r = idx
//     w   = clamp((t - st[l]) / ((st[r] - st[l]) + 1e-8f), 0, 1)
//     out = f[l] * (1 - w) + f[r] * w          (bf16 rows widened to fp32, one RN at the end)
// It replaces resample_trajectory_{bf16,fp32}_kernel
// (robocache/csrc/cuda/resample_kernel.cu:26-124) and multimodal_fusion_{fp32,bf16}_kernel
// (robocache/csrc/cuda/multimodal_kernel.cu:57-196).
#include <cuda_bf16.h>

#include "rc_common.cuh"

namespace {

constexpr int kMaxWarps = 8;       // warps per CTA at most
constexpr int kUnroll = 4;         // row vectors in flight per lane and source row
constexpr int kMaxStagedBytes = 200 * 1024;

struct StreamArg {
    const unsigned char* data;  // [B,S,D]
    const float* times;         // [B,S]
    long long row_bytes;        // D * element size
    long long col_bytes;        // byte offset of this stream's slice inside an output row
    int S;
    int vecs;                   // row_bytes / VEC
    int smem_off;               // float offset of the staged time row
    int pad_;
};

struct InterpParams {
    StreamArg s[RC_MAX_STREAMS];
    const float* tt;            // [B,T]
    unsigned char* out;         // [B,T,sum D]
    long long out_row_bytes;
    int ns;
    int T;
    int tiles_per_row;          // ceil(T / (32*W))
    int pad_;
};

// ---------------------------------------------------------------- bracket search

// count of a[0..n) strictly below t; n >= 1; same trip count in every lane
__device__ __forceinline__ int lower_bound(const float* a, int n, float t) {
    int base = 0;
    while (n > 1) {
        const int half = n >> 1;
        base += (a[base + half - 1] < t) ? half : 0;
        n -= half;
    }
    return base + ((a[base] < t) ? 1 : 0);
}

__device__ __forceinline__ void bracket(const float* a, int S, float t, int& l, int& r, float& w) {
    const int c = lower_bound(a, S, t);
    r = min(max(c, 1), S - 1);  // the upper bound wins when S == 1
    l = r - 1;
    if (l < 0) l += S;          // S == 1: both rows are row 0
    const float tl = a[l];
    const float tr = a[r];
    float q = __fdiv_rn(__fsub_rn(t, tl), __fadd_rn(__fsub_rn(tr, tl), 1e-8f));
    q = (q < 0.0f) ? 0.0f : ((q > 1.0f) ? 1.0f : q);  // NaN passes through, as torch.clamp
    w = q;
}

// ---------------------------------------------------------------- vector lerp

template <int VEC> struct VecOf;
template <> struct VecOf<16> { using type = uint4; };
template <> struct VecOf<8>  { using type = uint2; };
template <> struct VecOf<4>  { using type = unsigned int; };
template <> struct VecOf<2>  { using type = unsigned short; };

__device__ __forceinline__ float lerp1(float a, float b, float w, float om) {
    return __fadd_rn(__fmul_rn(a, om), __fmul_rn(b, w));
}

// one 32-bit word: a float (ES == 4) or two bf16 (ES == 2)
template <int ES>
__device__ __forceinline__ unsigned int lerp_word(unsigned int a, unsigned int b, float w, float om) {
    if (ES == 4) {
        return __float_as_uint(lerp1(__uint_as_float(a), __uint_as_float(b), w, om));
    } else {
        const float lo = lerp1(__uint_as_float(a << 16), __uint_as_float(b << 16), w, om);
        const float hi = lerp1(__uint_as_float(a & 0xffff0000u), __uint_as_float(b & 0xffff0000u), w, om);
        const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), .y = hi
        return *reinterpret_cast<const unsigned int*>(&p);
    }
}

template <int ES, int VEC>
__device__ __forceinline__ typename VecOf<VEC>::type lerp_vec(typename VecOf<VEC>::type a,
                                                              typename VecOf<VEC>::type b, float w, float om);

template <> __device__ __forceinline__ uint4 lerp_vec<2, 16>(uint4 a, uint4 b, float w, float om) {
    return make_uint4(lerp_word<2>(a.x, b.x, w, om), lerp_word<2>(a.y, b.y, w, om),
                      lerp_word<2>(a.z, b.z, w, om), lerp_word<2>(a.w, b.w, w, om));
}
template <> __device__ __forceinline__ uint4 lerp_vec<4, 16>(uint4 a, uint4 b, float w, float om) {
    return make_uint4(lerp_word<4>(a.x, b.x, w, om), lerp_word<4>(a.y, b.y, w, om),
                      lerp_word<4>(a.z, b.z, w, om), lerp_word<4>(a.w, b.w, w, om));
}
template <> __device__ __forceinline__ uint2 lerp_vec<2, 8>(uint2 a, uint2 b, float w, float om) {
    return make_uint2(lerp_word<2>(a.x, b.x, w, om), lerp_word<2>(a.y, b.y, w, om));
}
template <> __device__ __forceinline__ uint2 lerp_vec<4, 8>(uint2 a, uint2 b, float w, float om) {
    return make_uint2(lerp_word<4>(a.x, b.x, w, om), lerp_word<4>(a.y, b.y, w, om));
}
template <> __device__ __forceinline__ unsigned int lerp_vec<2, 4>(unsigned int a, unsigned int b, float w, float om) {
    return lerp_word<2>(a, b, w, om);
}
template <> __device__ __forceinline__ unsigned int lerp_vec<4, 4>(unsigned int a, unsigned int b, float w, float om) {
    return lerp_word<4>(a, b, w, om);
}
template <> __device__ __forceinline__ unsigned short lerp_vec<2, 2>(unsigned short a, unsigned short b, float w, float om) {
    const float v = lerp1(__uint_as_float(static_cast<unsigned int>(a) << 16),
                          __uint_as_float(static_cast<unsigned int>(b) << 16), w, om);
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    return *reinterpret_cast<const unsigned short*>(&h);
}

template <typename V> __device__ __forceinline__ V load_row(const unsigned char* p) {
    return __ldg(reinterpret_cast<const V*>(p));
}
template <typename V> __device__ __forceinline__ void store_row(unsigned char* p, V v) {
    __stcs(reinterpret_cast<V*>(p), v);  // the output is written once and never re-read here
}

// ---------------------------------------------------------------- one stream, one warp chunk

// Interpolates the rows of `nt` consecutive targets (owned by lanes 0..nt-1, which hold
// their bracket row `l` and weight `w`) of one stream into its output slice.
template <int ES, int VEC>
__device__ __forceinline__ void interp_chunk(const StreamArg& s, const unsigned char* src_b,
                                             unsigned char* out_t0, long long out_row_bytes,
                                             int l, float w, int nt, int lane) {
    using V = typename VecOf<VEC>::type;
    const int vecs = s.vecs;
    const int Sm1 = s.S - 1;
    if ((vecs & 31) == 0) {
        // rows of whole warps' width: the target index is uniform across the warp
        for (int j0 = 0; j0 < nt; j0 += kUnroll) {
            const unsigned char* pl[kUnroll];
            const unsigned char* pr[kUnroll];
            float wj[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int j = min(j0 + u, nt - 1);
                const int lj = __shfl_sync(0xffffffffu, l, j);
                wj[u] = __shfl_sync(0xffffffffu, w, j);
                pl[u] = src_b + static_cast<long long>(lj) * s.row_bytes;
                pr[u] = src_b + static_cast<long long>(min(lj + 1, Sm1)) * s.row_bytes;
            }
            for (int c = lane; c < vecs; c += 32) {
                V a[kUnroll], b[kUnroll];
                const long long cb = static_cast<long long>(c) * VEC;
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    if (j0 + u < nt) {
                        a[u] = load_row<V>(pl[u] + cb);
                        b[u] = load_row<V>(pr[u] + cb);
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    if (j0 + u < nt) {
                        const V o = lerp_vec<ES, VEC>(a[u], b[u], wj[u], __fsub_rn(1.0f, wj[u]));
                        store_row<V>(out_t0 + static_cast<long long>(j0 + u) * out_row_bytes + s.col_bytes + cb, o);
                    }
                }
            }
        }
    } else {
        // narrow or ragged rows: lanes walk the flat (target, vector) space
        const int total = nt * vecs;
        for (int v0 = 0; v0 < total; v0 += 32 * kUnroll) {
            V a[kUnroll], b[kUnroll];
            float wj[kUnroll];
            long long ob[kUnroll];
            bool ok[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int v = v0 + u * 32 + lane;
                ok[u] = v < total;
                const int j = ok[u] ? (v / vecs) : 0;
                const int c = ok[u] ? (v - j * vecs) : 0;
                const int lj = __shfl_sync(0xffffffffu, l, j);
                wj[u] = __shfl_sync(0xffffffffu, w, j);
                const long long cb = static_cast<long long>(c) * VEC;
                ob[u] = static_cast<long long>(j) * out_row_bytes + s.col_bytes + cb;
                if (ok[u]) {
                    a[u] = load_row<V>(src_b + static_cast<long long>(lj) * s.row_bytes + cb);
                    b[u] = load_row<V>(src_b + static_cast<long long>(min(lj + 1, Sm1)) * s.row_bytes + cb);
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (ok[u]) {
                    const V o = lerp_vec<ES, VEC>(a[u], b[u], wj[u], __fsub_rn(1.0f, wj[u]));
                    store_row<V>(out_t0 + ob[u], o);
                }
            }
        }
    }
}

// ---------------------------------------------------------------- kernel

// STAGED: timestamp rows live in shared memory; otherwise lanes search global memory
// (rows too long for shared memory).
template <int ES, int VEC, bool STAGED>
__global__ void __launch_bounds__(32 * kMaxWarps)
interp_kernel(const __grid_constant__ InterpParams p) {
    extern __shared__ __align__(16) float s_times[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const long long b = blockIdx.x / p.tiles_per_row;
    const int tile = static_cast<int>(blockIdx.x - b * p.tiles_per_row);

    if (STAGED) {
        for (int k = 0; k < p.ns; ++k) {
            const float* g = p.s[k].times + b * p.s[k].S;
            float* d = s_times + p.s[k].smem_off;
            for (int i = threadIdx.x; i < p.s[k].S; i += blockDim.x) d[i] = __ldg(g + i);
        }
        __syncthreads();
    }

    const int t0 = (tile * nwarps + warp) * 32;
    if (t0 >= p.T) return;
    const int nt = min(32, p.T - t0);
    const float tq = (lane < nt) ? __ldg(p.tt + b * p.T + t0 + lane) : 0.0f;
    unsigned char* out_t0 = p.out + (b * p.T + t0) * p.out_row_bytes;

    for (int k = 0; k < p.ns; ++k) {
        const StreamArg& s = p.s[k];
        const float* a = STAGED ? (s_times + s.smem_off) : (s.times + b * s.S);
        int l, r;
        float w;
        bracket(a, s.S, tq, l, r, w);
        (void)r;
        interp_chunk<ES, VEC>(s, s.data + b * s.S * s.row_bytes, out_t0, p.out_row_bytes, l, w, nt, lane);
    }
}

// brackets and weights only
__global__ void __launch_bounds__(256)
bracket_kernel(const float* __restrict__ st, const float* __restrict__ tt, long long B, int S, int T,
               int* __restrict__ left, int* __restrict__ right, float* __restrict__ weight) {
    const long long n = B * T;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long b = i / T;
        int l, r;
        float w;
        bracket(st + b * S, S, __ldg(tt + i), l, r, w);
        if (left) left[i] = l;
        if (right) right[i] = r;
        if (weight) weight[i] = w;
    }
}

// ---------------------------------------------------------------- host side

template <int ES, int VEC>
int launch_interp(const InterpParams& p, long long grid, int threads, size_t smem, bool staged,
                  cudaStream_t stream) {
    if (staged) {
        auto* k = interp_kernel<ES, VEC, true>;
        if (smem > 48 * 1024) {
            RC_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem)));
        }
        k<<<static_cast<unsigned int>(grid), threads, smem, stream>>>(p);
    } else {
        interp_kernel<ES, VEC, false><<<static_cast<unsigned int>(grid), threads, 0, stream>>>(p);
    }
    return rc::check_launch();
}

int interp_dispatch(const rc_stream_desc* streams, int ns, const float* tt, void* out, int64_t B,
                    int64_t T, int dtype, int device, void* stream_v) {
    if (dtype != RC_DTYPE_F32 && dtype != RC_DTYPE_BF16) return RC_ERR_BAD_DTYPE;
    if (ns < 1 || ns > RC_MAX_STREAMS) return RC_ERR_BAD_SHAPE;
    if (streams == nullptr) return RC_ERR_NULL_POINTER;
    if (B < 0 || T < 0) return RC_ERR_BAD_SHAPE;
    const int es = (dtype == RC_DTYPE_BF16) ? 2 : 4;

    long long out_d = 0;
    long long staged_floats = 0;
    for (int k = 0; k < ns; ++k) {
        if (streams[k].S < 0 || streams[k].D < 0) return RC_ERR_BAD_SHAPE;
        if (streams[k].S >= (1ll << 31) || streams[k].D >= (1ll << 31)) return RC_ERR_TOO_LARGE;
        out_d += streams[k].D;
        staged_floats += streams[k].S;
    }
    if (T >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (B == 0 || T == 0 || out_d == 0) return RC_OK;  // nothing to write
    for (int k = 0; k < ns; ++k) {
        if (streams[k].S == 0) return RC_ERR_BAD_SHAPE;  // no row to interpolate from
    }
    if (tt == nullptr || out == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(tt, 4) || !rc::aligned_to(out, es)) return RC_ERR_BAD_ALIGNMENT;

    InterpParams p{};
    p.ns = ns;
    p.tt = tt;
    p.out = static_cast<unsigned char*>(out);
    p.out_row_bytes = out_d * es;
    p.T = static_cast<int>(T);

    // widest access every row, slice and pointer allows
    uintptr_t bits = reinterpret_cast<uintptr_t>(out) | static_cast<uintptr_t>(p.out_row_bytes);
    long long col = 0;
    int smem_off = 0;
    int live = 0;
    for (int k = 0; k < ns; ++k) {
        if (streams[k].D == 0) continue;  // an empty slice contributes nothing
        if (streams[k].data == nullptr || streams[k].times == nullptr) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(streams[k].data, es) || !rc::aligned_to(streams[k].times, 4))
            return RC_ERR_BAD_ALIGNMENT;
        StreamArg& s = p.s[live++];
        s.data = static_cast<const unsigned char*>(streams[k].data);
        s.times = streams[k].times;
        s.S = static_cast<int>(streams[k].S);
        s.row_bytes = streams[k].D * es;
        s.col_bytes = col;
        s.smem_off = smem_off;
        smem_off += (s.S + 3) & ~3;  // keep every staged row 16-byte aligned
        bits |= reinterpret_cast<uintptr_t>(s.data) | static_cast<uintptr_t>(s.row_bytes) |
                static_cast<uintptr_t>(col);
        col += s.row_bytes;
    }
    p.ns = live;
    int vec = 16;
    while (vec > es && (bits & (vec - 1)) != 0) vec >>= 1;
    for (int k = 0; k < live; ++k) p.s[k].vecs = static_cast<int>(p.s[k].row_bytes / vec);

    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();

    // warps per CTA: enough to cover a target row, fewer when the grid would be too small
    int warps = 1;
    while (warps < kMaxWarps && warps * 32 < T) warps <<= 1;
    const long long want = 4ll * rc::sm_count(device);
    while (warps > 1 && B * ((T + 32 * warps - 1) / (32 * warps)) < want) warps >>= 1;
    p.tiles_per_row = static_cast<int>((T + 32 * warps - 1) / (32 * warps));
    const long long grid = B * p.tiles_per_row;
    if (grid >= (1ll << 31)) return RC_ERR_TOO_LARGE;

    const size_t smem = static_cast<size_t>(smem_off) * sizeof(float);
    const bool staged = smem <= static_cast<size_t>(kMaxStagedBytes);
    (void)staged_floats;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int threads = warps * 32;

    if (es == 2) {
        switch (vec) {
            case 16: return launch_interp<2, 16>(p, grid, threads, smem, staged, stream);
            case 8:  return launch_interp<2, 8>(p, grid, threads, smem, staged, stream);
            case 4:  return launch_interp<2, 4>(p, grid, threads, smem, staged, stream);
            default: return launch_interp<2, 2>(p, grid, threads, smem, staged, stream);
        }
    }
    switch (vec) {
        case 16: return launch_interp<4, 16>(p, grid, threads, smem, staged, stream);
        case 8:  return launch_interp<4, 8>(p, grid, threads, smem, staged, stream);
        default: return launch_interp<4, 4>(p, grid, threads, smem, staged, stream);
    }
}

}  // namespace

extern "C" {

int rc_resample(const void* src, const float* source_times, const float* target_times, void* out,
                int64_t B, int64_t S, int64_t T, int64_t D, int dtype, int device, void* stream) {
    rc_stream_desc s{src, source_times, S, D};
    return interp_dispatch(&s, 1, target_times, out, B, T, dtype, device, stream);
}

int rc_fuse(const rc_stream_desc* streams, int n_streams, const float* target_times, void* out,
            int64_t B, int64_t T, int dtype, int device, void* stream) {
    return interp_dispatch(streams, n_streams, target_times, out, B, T, dtype, device, stream);
}

int rc_resample_brackets(const float* source_times, const float* target_times, int64_t B, int64_t S,
                         int64_t T, int32_t* left, int32_t* right, float* weight, int device,
                         void* stream) {
    if (B < 0 || S < 0 || T < 0) return RC_ERR_BAD_SHAPE;
    if (S >= (1ll << 31) || T >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (B == 0 || T == 0) return RC_OK;
    if (S == 0) return RC_ERR_BAD_SHAPE;
    if (source_times == nullptr || target_times == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(source_times, 4) || !rc::aligned_to(target_times, 4) ||
        !rc::aligned_to(left, 4) || !rc::aligned_to(right, 4) || !rc::aligned_to(weight, 4))
        return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    const long long n = B * T;
    long long blocks = (n + 255) / 256;
    const long long cap = 32ll * rc::sm_count(device);
    if (blocks > cap) blocks = cap;
    bracket_kernel<<<static_cast<unsigned int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        source_times, target_times, B, static_cast<int>(S), static_cast<int>(T), left, right, weight);
    return rc::check_launch();
}

}  // extern "C"
