// Timestamp-aligned resampling and N-stream temporal fusion for sm_100a.
//
// Two kernels serve both operators; the host picks per call (interp_dispatch):
//   * the row-gather kernel below, for any shape (the resampling headline: rows of a long source
//     are fetched straight from global memory, only the rows that are used);
//   * the block kernel further down, when all inputs of one batch item fit in shared memory (the
//     fusion shapes): the item is staged whole with bulk asynchronous copies (TMA).
//
// Row-gather kernel.  A CTA owns one batch row b and a tile of 32*W
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

#include <atomic>

#include "rc_common.cuh"

namespace {

constexpr int kMaxWarps = 8;       // warps per CTA at most
constexpr int kMaxStagedBytes = 200 * 1024;

struct StreamArg {
    const unsigned char* data;  // [B,S,D], or packed rows [sum S_b, D] when row_offsets is set
    const float* times;         // [B,S], or packed [sum S_b]
    const long long* row_offsets;  // ragged input: item b owns rows [row_offsets[b], row_offsets[b+1]); else NULL
    long long time_stride;      // floats between the time rows of consecutive items (0: one row shared by all)
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
    long long tt_stride;        // floats between target rows of consecutive items (0: shared row)
    unsigned char* out;         // [B,T,sum D]
    long long out_row_bytes;
    int ns;
    int T;
    int tiles_per_row;          // ceil(T / (32*W))
    int bulk_stage;             // 1: the timestamp rows are staged by bulk asynchronous copies (RC_OPT_GATHER_BULK_STAGE)
    unsigned int wait_limit;    // polls of the wait for those copies (RC_OPT_BULK_WAIT_LIMIT)
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

// ---------------------------------------------------------------- gather kernel: one warp chunk

// Interpolates the rows of `nt` consecutive targets (owned by lanes 0..nt-1, which hold
// their bracket row `l` and weight `w`) of one stream into its output slice.
// UNIFORM: every row is a whole number of warp-wide accesses, so all lanes work on the
// same target and U targets are kept in flight; otherwise lanes walk the flat
// (target, vector) space of the chunk.
template <int ES, int VEC, bool UNIFORM, int U>
__device__ __forceinline__ void interp_chunk(const StreamArg& s, const unsigned char* src_b,
                                             unsigned char* out_t0, long long out_row_bytes,
                                             int S, int l, float w, int nt, int lane) {
    using V = typename VecOf<VEC>::type;
    const int vecs = s.vecs;
    const int Sm1 = S - 1;
    if (UNIFORM || (vecs & 31) == 0) {
        for (int j0 = 0; j0 < nt; j0 += U) {
            const unsigned char* pl[U];
            const unsigned char* pr[U];
            float wj[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = min(j0 + u, nt - 1);
                const int lj = __shfl_sync(0xffffffffu, l, j);
                wj[u] = __shfl_sync(0xffffffffu, w, j);
                pl[u] = src_b + static_cast<long long>(lj) * s.row_bytes;
                pr[u] = src_b + static_cast<long long>(min(lj + 1, Sm1)) * s.row_bytes;
            }
            for (int c = lane; c < vecs; c += 32) {
                V a[U], b[U];
                const long long cb = static_cast<long long>(c) * VEC;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (j0 + u < nt) {
                        a[u] = load_row<V>(pl[u] + cb);
                        b[u] = load_row<V>(pr[u] + cb);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (j0 + u < nt) {
                        const V o = lerp_vec<ES, VEC>(a[u], b[u], wj[u], __fsub_rn(1.0f, wj[u]));
                        store_row<V>(out_t0 + static_cast<long long>(j0 + u) * out_row_bytes + s.col_bytes + cb, o);
                    }
                }
            }
        }
    } else {
        const int total = nt * vecs;
        for (int v0 = 0; v0 < total; v0 += 32) {   // warp-uniform trip count: every lane reaches the shuffles
            const int v = v0 + lane;
            const bool ok = v < total;
            const int j = ok ? (v / vecs) : 0;
            const int c = ok ? (v - j * vecs) : 0;
            const int lj = __shfl_sync(0xffffffffu, l, j);
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (ok) {
                const long long cb = static_cast<long long>(c) * VEC;
                const V a = load_row<V>(src_b + static_cast<long long>(lj) * s.row_bytes + cb);
                const V b = load_row<V>(src_b + static_cast<long long>(min(lj + 1, Sm1)) * s.row_bytes + cb);
                const V o = lerp_vec<ES, VEC>(a, b, wj, __fsub_rn(1.0f, wj));
                store_row<V>(out_t0 + static_cast<long long>(j) * out_row_bytes + s.col_bytes + cb, o);
            }
        }
    }
}

// ---------------------------------------------------------------- gather kernel

constexpr unsigned int kMbarSpinLimit = 1u << 22;

// how often a CTA gave up waiting for its bulk copies and fetched the data with plain loads
__device__ unsigned int g_bulk_wait_timeouts = 0;

__device__ __forceinline__ unsigned int smem_u32(const void* p) {
    return static_cast<unsigned int>(__cvta_generic_to_shared(p));
}
// shared-memory loads through 32-bit window addresses (results of smem_u32)
__device__ __forceinline__ unsigned int lds_u32(unsigned int addr) {
    unsigned int v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32(unsigned int addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(unsigned int addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one thread: global -> this CTA's shared memory, completion counted in bytes on `bar`
// (no multicast: source and destination belong to this GPU and this CTA)
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, unsigned int bytes,
                                          unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// bounded wait on phase `parity`: at most `limit` polls; false if they ran out
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned int parity, unsigned int limit) {
    const unsigned int addr = smem_u32(bar);
    for (unsigned int i = 0; i < limit; ++i) {
        unsigned int done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}

// STAGED: timestamp rows live in shared memory; otherwise lanes search global memory
// (rows too long for shared memory).  Four CTAs of 256 threads per SM (64 registers).
template <int ES, int VEC, bool STAGED, bool UNIFORM, bool RAGGED>
__global__ void __launch_bounds__(32 * kMaxWarps, 4)
interp_gather_kernel(const __grid_constant__ InterpParams p) {
    extern __shared__ __align__(16) float s_times[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const long long b = blockIdx.x / p.tiles_per_row;
    const int tile = static_cast<int>(blockIdx.x - b * p.tiles_per_row);

    // item b of stream k: first row and number of rows (dense: b*S and S)
    auto first_row = [&](int k) -> long long {
        return RAGGED ? __ldg(p.s[k].row_offsets + b) : b * p.s[k].S;
    };
    // ragged: the caller's bound max_len (held in S) sized the staged row, so an item that is longer than
    // that, or offsets that do not ascend, are cut to [0, max_len] rows instead of running past the staging
    auto num_rows = [&](int k) -> int {
        if (!RAGGED) return p.s[k].S;
        const long long n = __ldg(p.s[k].row_offsets + b + 1) - __ldg(p.s[k].row_offsets + b);
        return static_cast<int>(n < 0 ? 0 : (n > p.s[k].S ? p.s[k].S : n));
    };

    __shared__ __align__(8) unsigned long long bar;
    bool gave_up = false;       // thread 0 only: its bounded wait for the bulk copies ran out
    if (STAGED) {
        bool staged = false;
        if (!RAGGED && p.bulk_stage) {
            // one thread fetches every time row with a bulk asynchronous copy (TMA) and waits for it, bounded;
            // should the wait run out, the rows are fetched again with ordinary loads below
            bool arrived = true;
            if (threadIdx.x == 0) {
                unsigned int bytes = 0;
                for (int k = 0; k < p.ns; ++k) bytes += static_cast<unsigned int>(p.s[k].S) * 4u;
                mbar_init(&bar, 1);
                mbar_expect_tx(&bar, bytes);
                for (int k = 0; k < p.ns; ++k)
                    bulk_load(s_times + p.s[k].smem_off, p.s[k].times + b * p.s[k].time_stride,
                              static_cast<unsigned int>(p.s[k].S) * 4u, &bar);
                arrived = mbar_wait(&bar, 0, p.wait_limit);
                if (!arrived) atomicAdd(&g_bulk_wait_timeouts, 1u);
                gave_up = !arrived;
            }
            staged = !__syncthreads_or(!arrived);
        }
        if (!staged) {
            for (int k = 0; k < p.ns; ++k) {
                const float* g = p.s[k].times + (RAGGED ? first_row(k) : b * p.s[k].time_stride);
                float* d = s_times + p.s[k].smem_off;
                const int n = num_rows(k);
                for (int i = threadIdx.x; i < n; i += blockDim.x) d[i] = __ldg(g + i);
            }
            __syncthreads();
        }
    }

    const int t0 = (tile * nwarps + warp) * 32;
    if (t0 >= p.T) return;
    const int nt = min(32, p.T - t0);
    const float tq = (lane < nt) ? __ldg(p.tt + b * p.tt_stride + t0 + lane) : 0.0f;
    unsigned char* out_t0 = p.out + (b * p.T + t0) * p.out_row_bytes;

    for (int k = 0; k < p.ns; ++k) {
        const StreamArg& s = p.s[k];
        const long long row0 = first_row(k);
        const int S = num_rows(k);
        if (RAGGED && S <= 0) {
            // an item without source rows yields zeros
            for (int i = lane; i < nt * static_cast<int>(s.row_bytes); i += 32) {
                const int j = i / static_cast<int>(s.row_bytes);
                out_t0[static_cast<long long>(j) * p.out_row_bytes + s.col_bytes + (i - j * static_cast<int>(s.row_bytes))] = 0;
            }
            continue;
        }
        const float* a = STAGED ? (s_times + s.smem_off) : (s.times + (RAGGED ? row0 : b * s.time_stride));
        int l, r;
        float w;
        bracket(a, S, tq, l, r, w);
        (void)r;
        interp_chunk<ES, VEC, UNIFORM, UNIFORM ? 2 : 1>(s, s.data + row0 * s.row_bytes, out_t0,
                                                        p.out_row_bytes, S, l, w, nt, lane);
    }
    // a CTA that gave up on its bulk copies must not hand its shared memory on while they may still land
    if (gave_up) mbar_wait(&bar, 0, kMbarSpinLimit);
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

// ---------------------------------------------------------------- block kernel (TMA-staged inputs)
//
// When the inputs of one batch item are small enough to sit in shared memory (the fusion
// shapes: 48 KB for 30x512 + 100x64 + 200x12 bf16) a CTA fetches them whole with one bulk
// asynchronous copy (TMA, cp.async.bulk) per stream, completes them on an mbarrier, and
// computes its output rows out of shared memory.  Global memory then sees only large
// contiguous reads (every input byte exactly once per CTA) and fully coalesced writes;
// rows narrower than a warp access (24-byte IMU rows) and output rows that are only
// 8-byte aligned cost nothing extra.  Work is cut into 8-byte pieces of output rows (4 bf16
// or 2 fp32), written two at a time as 16-byte vectors where the row geometry allows, so
// every stream width must be a multiple of 8 bytes.

constexpr int kBlockThreads = 512;  // 4 CTAs x 16 warps per SM at the fusion headline shape (measured best of 256/512/1024)
constexpr int kBlockSmemLimit = 100 * 1024;     // keeps at least two CTAs per SM

struct BlockStream {
    const unsigned char* data;
    const float* times;
    int S;
    int row_bytes;
    int half_off;       // first 8-byte piece of this stream inside an output row
    int data_off;       // byte offset of the staged data in shared memory
    int time_off;       // float offset of the staged time row
    int block_bytes;    // S * row_bytes
    long long time_stride;  // floats between the time rows of consecutive items (0: shared row)
};

struct BlockParams {
    BlockStream s[RC_MAX_STREAMS];
    const float* tt;
    long long tt_stride;        // floats between target rows of consecutive items (0: shared row)
    unsigned char* out;
    long long out_block_bytes;  // T * out_row_bytes
    int out_row_bytes;
    int hpr;                    // 8-byte pieces per output row
    int ns;
    int T;
    int tiles_t;
    int rows_per_tile;
    int times_base;             // byte offsets of the regions after the staged data
    int brk_base;
    int vec_base;               // table of output-vector descriptors (16-byte path)
    unsigned int tx_bytes;      // sum of block_bytes
    unsigned int wait_limit;    // polls of the first wait for the bulk copies (RC_OPT_BULK_WAIT_LIMIT)
};

// pieces of the block kernel ---------------------------------------------------------------

// brackets of rows [t_begin, t_begin + nrows) of item b, one (stream, row) pair per thread, stored as
// byte offsets (from the stage origin) of the two bracket rows, plus the weight
__device__ __forceinline__ void block_brackets(const BlockParams& p, const float* s_times, int* s_lo, int* s_hi,
                                               float* s_w, long long b, int t_begin, int nrows, int tid, int nthreads) {
    for (int i = tid; i < nrows * p.ns; i += nthreads) {
        const int k = i / nrows;
        const int r = i - k * nrows;
        const BlockStream& s = p.s[k];
        int l, rr;
        float w;
        bracket(s_times + s.time_off, s.S, __ldg(p.tt + b * p.tt_stride + t_begin + r), l, rr, w);
        s_lo[k * p.rows_per_tile + r] = s.data_off + l * s.row_bytes;
        s_hi[k * p.rows_per_tile + r] = s.data_off + rr * s.row_bytes;
        s_w[k * p.rows_per_tile + r] = w;
    }
}

// the same bytes a bulk copy would have delivered, fetched with ordinary loads (a wait timed out)
__device__ __forceinline__ void block_fetch_plain(const BlockParams& p, unsigned char* stage, long long b, int tid,
                                                  int nthreads) {
    for (int k = 0; k < p.ns; ++k) {
        const uint2* g = reinterpret_cast<const uint2*>(p.s[k].data + b * p.s[k].block_bytes);
        uint2* d = reinterpret_cast<uint2*>(stage + p.s[k].data_off);
        for (int i = tid; i < p.s[k].block_bytes / 8; i += nthreads) d[i] = __ldg(g + i);
    }
}

// Descriptor table (offsets relative to the stage origin).  16-byte path: for each vector of a row
// group and each of its two 8-byte halves, the offset of its piece inside a staged row (x, y) and the
// offset of its bracket entry for group 0 (z, w).  8-byte path: the same for each piece of a row (x, z).
template <bool V16>
__device__ __forceinline__ void block_unit_table(const BlockParams& p, uint4* s_vec, int tid, int nthreads) {
    const int G = (V16 && (p.hpr & 1)) ? 2 : 1;
    const int units = V16 ? ((G * p.hpr) >> 1) : p.hpr;
    for (int m = tid; m < units; m += nthreads) {
        unsigned int e[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int h = 0; h < (V16 ? 2 : 1); ++h) {
            const int q = V16 ? (2 * m + h) : m;
            const int dr = (q >= p.hpr) ? 1 : 0;
            const int c = q - dr * p.hpr;
            int k = 0;
            for (int j = 1; j < p.ns; ++j) k += (c >= p.s[j].half_off) ? 1 : 0;
            e[h] = static_cast<unsigned int>((c - p.s[k].half_off) * 8);
            e[2 + h] = static_cast<unsigned int>(p.brk_base) + static_cast<unsigned int>(k * p.rows_per_tile + dr) * 4u;
        }
        s_vec[m] = make_uint4(e[0], e[1], e[2], e[3]);
    }
}

// Interpolates `nrows` rows of one item out of a stage into out_tile.
// V16: output written as 16-byte vectors.  Output rows are a multiple of 8 bytes, so rows (or, when a
// row is an odd number of 8-byte pieces, pairs of rows) start 16-byte aligned; a group of G = 1 or 2
// rows is then a whole number of vectors, and which (row of the group, piece) each half of vector m
// covers is the same for every group: it is read from the descriptor table, and the threads walk the
// flat (group, vector) space of the tile, so the work is spread evenly whatever the row width.
// Otherwise the unit is an 8-byte piece of a row, walked the same way over the flat (row, piece) space.
template <int ES, bool V16>
__device__ __forceinline__ void block_compute(const BlockParams& p, const unsigned char* stage, const uint4* s_vec,
                                              unsigned char* out_tile, int nrows, int tid, int nthreads) {
    const int* s_lo = reinterpret_cast<const int*>(stage + p.brk_base);
    const int* s_hi = s_lo + p.ns * p.rows_per_tile;
    const float* s_w = reinterpret_cast<const float*>(s_hi + p.ns * p.rows_per_tile);
    if (V16) {
        const int G = (p.hpr & 1) ? 2 : 1;
        const int vpg = (G * p.hpr) >> 1;             // vectors per group
        const int ngroups = nrows / G;                // the host guarantees nrows % G == 0
        const unsigned int sb = smem_u32(stage);
        const unsigned int plane = static_cast<unsigned int>(p.ns * p.rows_per_tile) * 4u;  // lo -> hi -> w arrays
        const int total = ngroups * vpg;
        const int dm = nthreads % vpg, dg = nthreads / vpg;
        int m = tid % vpg, g = tid / vpg;
        const unsigned int gstep = static_cast<unsigned int>(G) * 4u;
        for (int v = tid; v < total; v += nthreads) {
            const uint4 e = s_vec[m];
            const unsigned int b0 = sb + e.z + static_cast<unsigned int>(g) * gstep;
            const unsigned int b1 = sb + e.w + static_cast<unsigned int>(g) * gstep;
            const unsigned int la = lds_u32(b0), ha = lds_u32(b0 + plane);
            const float wa = lds_f32(b0 + 2u * plane);
            unsigned int lb = la, hb = ha;
            float wb = wa;
            if (b1 != b0) {  // the halves lie in different rows or streams
                lb = lds_u32(b1); hb = lds_u32(b1 + plane); wb = lds_f32(b1 + 2u * plane);
            }
            const uint2 o0 = lerp_vec<ES, 8>(lds_v2(sb + e.x + la), lds_v2(sb + e.x + ha), wa, __fsub_rn(1.0f, wa));
            const uint2 o1 = lerp_vec<ES, 8>(lds_v2(sb + e.y + lb), lds_v2(sb + e.y + hb), wb, __fsub_rn(1.0f, wb));
            __stcs(reinterpret_cast<uint4*>(out_tile + static_cast<long long>(g) * (G * p.out_row_bytes) + m * 16),
                   make_uint4(o0.x, o0.y, o1.x, o1.y));
            m += dm; g += dg;
            if (m >= vpg) { m -= vpg; ++g; }
        }
    } else {
        const unsigned int sb = smem_u32(stage);
        const unsigned int plane = static_cast<unsigned int>(p.ns * p.rows_per_tile) * 4u;
        const int total = nrows * p.hpr;
        const int dm = nthreads % p.hpr, dg = nthreads / p.hpr;
        int m = tid % p.hpr, r = tid / p.hpr;
        for (int v = tid; v < total; v += nthreads) {
            const uint4 e = s_vec[m];
            const unsigned int b0 = sb + e.z + static_cast<unsigned int>(r) * 4u;
            const unsigned int la = lds_u32(b0), ha = lds_u32(b0 + plane);
            const float w = lds_f32(b0 + 2u * plane);
            const uint2 o = lerp_vec<ES, 8>(lds_v2(sb + e.x + la), lds_v2(sb + e.x + ha), w, __fsub_rn(1.0f, w));
            __stcs(reinterpret_cast<uint2*>(out_tile + static_cast<long long>(r) * p.out_row_bytes + m * 8), o);
            m += dm; r += dg;
            if (m >= p.hpr) { m -= p.hpr; ++r; }
        }
    }
}

// One CTA per (item, row tile).  With few items an item's rows spread over several CTAs (each stages
// the whole item; L2 serves the repeats).
template <int ES, bool V16>
__global__ void __launch_bounds__(kBlockThreads)
interp_block_kernel(const __grid_constant__ BlockParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(smem);
    float* s_times = reinterpret_cast<float*>(smem + p.times_base);
    int* s_lo = reinterpret_cast<int*>(smem + p.brk_base);
    int* s_hi = s_lo + p.ns * p.rows_per_tile;
    float* s_w = reinterpret_cast<float*>(s_hi + p.ns * p.rows_per_tile);
    uint4* s_vec = reinterpret_cast<uint4*>(smem + p.vec_base);

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;  // 512 for throughput, 256 when an item is split over several CTAs
    const long long b = blockIdx.x / p.tiles_t;
    const int tile = static_cast<int>(blockIdx.x - b * p.tiles_t);
    const int t_begin = tile * p.rows_per_tile;
    const int nrows = min(p.rows_per_tile, p.T - t_begin);

    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_expect_tx(bar, p.tx_bytes);
        for (int k = 0; k < p.ns; ++k)
            bulk_load(smem + p.s[k].data_off, p.s[k].data + b * p.s[k].block_bytes,
                      static_cast<unsigned int>(p.s[k].block_bytes), bar);
    }
    for (int k = 0; k < p.ns; ++k) {
        const float* g = p.s[k].times + b * p.s[k].time_stride;
        float* d = s_times + p.s[k].time_off;
        for (int i = tid; i < p.s[k].S; i += nthreads) d[i] = __ldg(g + i);
    }
    block_unit_table<V16>(p, s_vec, tid, nthreads);
    __syncthreads();  // mbarrier initialised, time rows visible
    block_brackets(p, s_times, s_lo, s_hi, s_w, b, t_begin, nrows, tid, nthreads);

    // One thread waits for the staged data (bounded); the others park at the barrier.  A CTA
    // whose wait runs out records it and fetches the same bytes with ordinary loads instead
    // (a late bulk copy only rewrites equal values while this CTA still owns the shared memory).
    bool arrived = true;
    if (tid == 0) arrived = mbar_wait(bar, 0, p.wait_limit);
    const bool gave_up = __syncthreads_or(!arrived);
    if (gave_up) {
        if (tid == 0) atomicAdd(&g_bulk_wait_timeouts, 1u);
        block_fetch_plain(p, smem, b, tid, nthreads);
        __syncthreads();
    }
    unsigned char* out_tile = p.out + b * p.out_block_bytes + static_cast<long long>(t_begin) * p.out_row_bytes;
    block_compute<ES, V16>(p, smem, s_vec, out_tile, nrows, tid, nthreads);
    if (gave_up) {
        // The copies may still be in flight: the CTA must not hand its shared memory to the next CTA on this SM
        // before they have landed.  Wait again, with the full limit; if even that runs out (a copy that never
        // completes), the CTA leaves, and the count above is what tells the host.
        if (tid == 0) mbar_wait(bar, 0, kMbarSpinLimit);
        __syncthreads();
    }
}

// ---------------------------------------------------------------- host side

template <int ES, int VEC, bool STAGED, bool UNIFORM>
int launch_gather_one(const InterpParams& p, unsigned int g, int threads, size_t smem, bool ragged, cudaStream_t stream) {
    if (STAGED && smem > 48 * 1024) {
        int device = 0;
        RC_CUDA_TRY(cudaGetDevice(&device));
        const void* k = ragged ? reinterpret_cast<const void*>(interp_gather_kernel<ES, VEC, STAGED, UNIFORM, true>)
                               : reinterpret_cast<const void*>(interp_gather_kernel<ES, VEC, STAGED, UNIFORM, false>);
        const int rc_attr = rc::ensure_dynamic_smem(k, device, smem);
        if (rc_attr != RC_OK) return rc_attr;
    }
    const size_t dyn = STAGED ? smem : 0;
    if (ragged) interp_gather_kernel<ES, VEC, STAGED, UNIFORM, true><<<g, threads, dyn, stream>>>(p);
    else        interp_gather_kernel<ES, VEC, STAGED, UNIFORM, false><<<g, threads, dyn, stream>>>(p);
    return rc::check_launch();
}

template <int ES, int VEC>
int launch_gather(const InterpParams& p, long long grid, int threads, size_t smem, bool staged, bool uniform,
                  cudaStream_t stream) {
    const unsigned int g = static_cast<unsigned int>(grid);
    const bool ragged = p.s[0].row_offsets != nullptr;
    if (staged) {
        return uniform ? launch_gather_one<ES, VEC, true, true>(p, g, threads, smem, ragged, stream)
                       : launch_gather_one<ES, VEC, true, false>(p, g, threads, smem, ragged, stream);
    }
    return uniform ? launch_gather_one<ES, VEC, false, true>(p, g, threads, smem, ragged, stream)
                   : launch_gather_one<ES, VEC, false, false>(p, g, threads, smem, ragged, stream);
}

struct LiveStream {
    const unsigned char* data;
    const float* times;
    long long S;
    long long row_bytes;
    long long time_stride;
};

// The TMA-staged block kernel applies when every stream width is a multiple of 8 bytes, every
// per-item input block can be bulk-copied (16-byte aligned, multiple of 16 bytes), the inputs
// of one item fit the shared-memory budget and most of them are actually used.
bool try_launch_block(const LiveStream* ls, int ns, const float* tt, long long tt_stride, unsigned char* out, long long B,
                      long long T, int es, int device, cudaStream_t stream, int* status) {
    BlockParams p{};
    long long in_bytes = 0, out_row = 0;
    int data_off = 16, time_off = 0;
    for (int k = 0; k < ns; ++k) {
        const long long blk = ls[k].S * ls[k].row_bytes;
        if ((ls[k].row_bytes & 7) != 0 || (blk & 15) != 0 || !rc::aligned_to(ls[k].data, 16)) return false;
        if (blk > kBlockSmemLimit) return false;
        BlockStream& s = p.s[k];
        s.data = ls[k].data;
        s.times = ls[k].times;
        s.time_stride = ls[k].time_stride;
        s.S = static_cast<int>(ls[k].S);
        s.row_bytes = static_cast<int>(ls[k].row_bytes);
        s.half_off = static_cast<int>(out_row / 8);
        s.data_off = data_off;
        s.time_off = time_off;
        s.block_bytes = static_cast<int>(blk);
        data_off += static_cast<int>(blk);
        time_off += static_cast<int>(ls[k].S);
        in_bytes += blk;
        out_row += ls[k].row_bytes;
        if (data_off > kBlockSmemLimit) return false;
    }
    if (!rc::aligned_to(out, 8) || out_row > (1 << 20)) return false;
    if (in_bytes > 2 * T * out_row) return false;  // mostly unused inputs: gathering rows moves fewer bytes
    // rows per CTA: whole items when there are plenty of them, slices of an item otherwise
    const int sms = rc::sm_count(device);
    long long tiles = 1;
    if (B < 2ll * sms) {
        tiles = (2ll * sms + B - 1) / B;
        const long long max_tiles = (T + 7) / 8;  // at least one row per warp
        if (tiles > max_tiles) tiles = max_tiles;
    }
    long long rpt = (T + tiles - 1) / tiles;
    // 16-byte output vectors: rows (or pairs of rows, when a row is an odd number of 8-byte pieces) must
    // start 16-byte aligned in every tile of every item
    const long long G = ((out_row / 8) & 1) ? 2 : 1;
    const bool v16 = rc::aligned_to(out, 16) && (T % G == 0);
    if (v16 && (rpt % G) != 0) ++rpt;
    tiles = (T + rpt - 1) / rpt;
    p.times_base = (data_off + 15) & ~15;
    p.brk_base = p.times_base + ((time_off * 4 + 15) & ~15);
    p.vec_base = static_cast<int>((p.brk_base + rpt * ns * 12 + 15) & ~15ll);
    const long long smem = p.vec_base + (v16 ? (G * (out_row / 8) / 2) : (out_row / 8)) * 16;
    if (smem > kBlockSmemLimit || B * tiles >= (1ll << 31)) return false;
    p.tt = tt;
    p.tt_stride = tt_stride;
    p.out = out;
    p.out_block_bytes = T * out_row;
    p.out_row_bytes = static_cast<int>(out_row);
    p.hpr = static_cast<int>(out_row / 8);
    p.ns = ns;
    p.T = static_cast<int>(T);
    p.tiles_t = static_cast<int>(tiles);
    p.rows_per_tile = static_cast<int>(rpt);
    p.tx_bytes = static_cast<unsigned int>(in_bytes);
    {
        const int opt = rc::g_bulk_wait_limit.load(std::memory_order_relaxed);
        p.wait_limit = opt < 0 ? kMbarSpinLimit : static_cast<unsigned int>(opt);
    }
    auto* kern = (es == 2) ? (v16 ? interp_block_kernel<2, true> : interp_block_kernel<2, false>)
                           : (v16 ? interp_block_kernel<4, true> : interp_block_kernel<4, false>);
    if (smem > 48 * 1024) {
        const int rc_attr = rc::ensure_dynamic_smem(reinterpret_cast<const void*>(kern), device, static_cast<size_t>(smem));
        if (rc_attr != RC_OK) { *status = rc_attr; return true; }
    }
    const int threads = (tiles > 1) ? 256 : kBlockThreads;  // split items are latency bound: smaller CTAs start sooner
    kern<<<static_cast<unsigned int>(B * tiles), threads, static_cast<size_t>(smem), stream>>>(p);
    *status = rc::check_launch();
    return true;
}

// time_strides: per stream, floats between the time rows of consecutive items (NULL: dense, = S); tt_stride: the
// same for the target rows (< 0: dense, = T).  A stride of 0 means one row shared by the whole batch.
int interp_dispatch(const rc_stream_desc* streams, int ns, const int64_t* time_strides, const float* tt,
                    int64_t tt_stride_in, void* out, int64_t B, int64_t T, int dtype, int device, void* stream_v) {
    if (dtype != RC_DTYPE_F32 && dtype != RC_DTYPE_BF16) return RC_ERR_BAD_DTYPE;
    if (ns < 1 || ns > RC_MAX_STREAMS) return RC_ERR_BAD_SHAPE;
    if (streams == nullptr) return RC_ERR_NULL_POINTER;
    if (B < 0 || T < 0) return RC_ERR_BAD_SHAPE;
    const int es = (dtype == RC_DTYPE_BF16) ? 2 : 4;

    long long out_d = 0;
    for (int k = 0; k < ns; ++k) {
        if (streams[k].S < 0 || streams[k].D < 0) return RC_ERR_BAD_SHAPE;
        if (streams[k].S >= (1ll << 31) || streams[k].D >= (1ll << 31)) return RC_ERR_TOO_LARGE;
        out_d += streams[k].D;
    }
    if (T >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (B == 0 || T == 0 || out_d == 0) return RC_OK;  // nothing to write
    for (int k = 0; k < ns; ++k) {
        if (streams[k].S == 0) return RC_ERR_BAD_SHAPE;  // no row to interpolate from
    }
    if (tt == nullptr || out == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(tt, 4) || !rc::aligned_to(out, es)) return RC_ERR_BAD_ALIGNMENT;

    // streams with D == 0 own an empty column slice and are dropped here
    LiveStream ls[RC_MAX_STREAMS];
    int live = 0;
    for (int k = 0; k < ns; ++k) {
        if (streams[k].D == 0) continue;
        if (streams[k].data == nullptr || streams[k].times == nullptr) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(streams[k].data, es) || !rc::aligned_to(streams[k].times, 4))
            return RC_ERR_BAD_ALIGNMENT;
        const long long ts = time_strides ? time_strides[k] : streams[k].S;
        if (ts != 0 && ts < streams[k].S) return RC_ERR_BAD_SHAPE;
        ls[live++] = LiveStream{static_cast<const unsigned char*>(streams[k].data), streams[k].times,
                                streams[k].S, streams[k].D * es, ts};
    }

    const long long tt_stride = (tt_stride_in < 0) ? T : tt_stride_in;
    if (tt_stride != 0 && tt_stride < T) return RC_ERR_BAD_SHAPE;

    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    if (rc::g_allow_block_kernel.load(std::memory_order_relaxed)) {
        int status = RC_OK;
        if (try_launch_block(ls, live, tt, tt_stride, static_cast<unsigned char*>(out), B, T, es, device, stream, &status))
            return status;
    }

    InterpParams p{};
    p.ns = live;
    p.tt = tt;
    p.tt_stride = tt_stride;
    p.out = static_cast<unsigned char*>(out);
    p.out_row_bytes = out_d * es;
    p.T = static_cast<int>(T);
    // widest access every row, slice and pointer allows
    uintptr_t bits = reinterpret_cast<uintptr_t>(out) | static_cast<uintptr_t>(p.out_row_bytes);
    long long col = 0;
    int smem_off = 0;
    for (int k = 0; k < live; ++k) {
        StreamArg& s = p.s[k];
        s.data = ls[k].data;
        s.times = ls[k].times;
        s.time_stride = ls[k].time_stride;
        s.S = static_cast<int>(ls[k].S);
        s.row_bytes = ls[k].row_bytes;
        s.col_bytes = col;
        s.smem_off = smem_off;
        smem_off += (s.S + 3) & ~3;  // keep every staged row 16-byte aligned
        bits |= reinterpret_cast<uintptr_t>(s.data) | static_cast<uintptr_t>(s.row_bytes) | static_cast<uintptr_t>(col);
        col += s.row_bytes;
    }
    int vec = 16;
    while (vec > es && (bits & (vec - 1)) != 0) vec >>= 1;
    bool uniform = true;
    for (int k = 0; k < live; ++k) {
        p.s[k].vecs = static_cast<int>(p.s[k].row_bytes / vec);
        uniform = uniform && (p.s[k].vecs % 32 == 0);
    }

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
    const int threads = warps * 32;
    // bulk-copy staging of the time rows: every row a whole number of 16-byte pieces at a 16-byte aligned address
    p.bulk_stage = 0;
    if (staged && rc::g_gather_bulk_stage.load(std::memory_order_relaxed)) {
        bool ok = true;
        for (int k = 0; k < live; ++k)
            ok = ok && (p.s[k].S % 4 == 0) && rc::aligned_to(p.s[k].times, 16) && (p.s[k].time_stride % 4 == 0);
        p.bulk_stage = ok ? 1 : 0;
        const int opt = rc::g_bulk_wait_limit.load(std::memory_order_relaxed);
        p.wait_limit = opt < 0 ? kMbarSpinLimit : static_cast<unsigned int>(opt);
    }
    if (es == 2) {
        switch (vec) {
            case 16: return launch_gather<2, 16>(p, grid, threads, smem, staged, uniform, stream);
            case 8:  return launch_gather<2, 8>(p, grid, threads, smem, staged, uniform, stream);
            case 4:  return launch_gather<2, 4>(p, grid, threads, smem, staged, uniform, stream);
            default: return launch_gather<2, 2>(p, grid, threads, smem, staged, uniform, stream);
        }
    }
    switch (vec) {
        case 16: return launch_gather<4, 16>(p, grid, threads, smem, staged, uniform, stream);
        case 8:  return launch_gather<4, 8>(p, grid, threads, smem, staged, uniform, stream);
        default: return launch_gather<4, 4>(p, grid, threads, smem, staged, uniform, stream);
    }
}

// Ragged resampling: one stream whose items have different lengths, packed back to back.
int ragged_dispatch(const void* src, const float* times, const long long* row_offsets, long long max_len,
                    const float* tt, void* out, int64_t B, int64_t T, int64_t D, int dtype, int device, void* stream_v) {
    if (dtype != RC_DTYPE_F32 && dtype != RC_DTYPE_BF16) return RC_ERR_BAD_DTYPE;
    if (B < 0 || T < 0 || D < 0 || max_len < 0) return RC_ERR_BAD_SHAPE;
    if (T >= (1ll << 31) || D >= (1ll << 31) || max_len >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (B == 0 || T == 0 || D == 0) return RC_OK;
    if (row_offsets == nullptr || tt == nullptr || out == nullptr) return RC_ERR_NULL_POINTER;
    if (max_len > 0 && (src == nullptr || times == nullptr)) return RC_ERR_NULL_POINTER;
    const int es = (dtype == RC_DTYPE_BF16) ? 2 : 4;
    if (!rc::aligned_to(src, es) || !rc::aligned_to(times, 4) || !rc::aligned_to(tt, 4) || !rc::aligned_to(out, es) ||
        !rc::aligned_to(row_offsets, 8))
        return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();

    InterpParams p{};
    p.ns = 1;
    p.tt = tt;
    p.tt_stride = T;
    p.out = static_cast<unsigned char*>(out);
    p.out_row_bytes = D * es;
    p.T = static_cast<int>(T);
    StreamArg& s = p.s[0];
    s.data = static_cast<const unsigned char*>(src);
    s.times = times;
    s.row_offsets = row_offsets;
    s.S = static_cast<int>(max_len);
    s.row_bytes = D * es;
    s.col_bytes = 0;
    s.smem_off = 0;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(s.row_bytes);
    int vec = 16;
    while (vec > es && (bits & (vec - 1)) != 0) vec >>= 1;
    s.vecs = static_cast<int>(s.row_bytes / vec);
    const bool uniform = (s.vecs % 32 == 0);
    int warps = 1;
    while (warps < kMaxWarps && warps * 32 < T) warps <<= 1;
    const long long want = 4ll * rc::sm_count(device);
    while (warps > 1 && B * ((T + 32 * warps - 1) / (32 * warps)) < want) warps >>= 1;
    p.tiles_per_row = static_cast<int>((T + 32 * warps - 1) / (32 * warps));
    const long long grid = B * p.tiles_per_row;
    if (grid >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    const size_t smem = static_cast<size_t>((max_len + 3) & ~3ll) * sizeof(float);
    const bool staged = smem <= static_cast<size_t>(kMaxStagedBytes);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int threads = warps * 32;
    if (es == 2) {
        switch (vec) {
            case 16: return launch_gather<2, 16>(p, grid, threads, smem, staged, uniform, stream);
            case 8:  return launch_gather<2, 8>(p, grid, threads, smem, staged, uniform, stream);
            case 4:  return launch_gather<2, 4>(p, grid, threads, smem, staged, uniform, stream);
            default: return launch_gather<2, 2>(p, grid, threads, smem, staged, uniform, stream);
        }
    }
    switch (vec) {
        case 16: return launch_gather<4, 16>(p, grid, threads, smem, staged, uniform, stream);
        case 8:  return launch_gather<4, 8>(p, grid, threads, smem, staged, uniform, stream);
        default: return launch_gather<4, 4>(p, grid, threads, smem, staged, uniform, stream);
    }
}

}  // namespace

extern "C" {

int rc_resample(const void* src, const float* source_times, const float* target_times, void* out,
                int64_t B, int64_t S, int64_t T, int64_t D, int dtype, int device, void* stream) {
    rc_stream_desc s{src, source_times, S, D};
    return interp_dispatch(&s, 1, nullptr, target_times, -1, out, B, T, dtype, device, stream);
}

int rc_resample_strided(const void* src, const float* source_times, int64_t source_time_stride,
                        const float* target_times, int64_t target_time_stride, void* out, int64_t B, int64_t S, int64_t T,
                        int64_t D, int dtype, int device, void* stream) {
    rc_stream_desc s{src, source_times, S, D};
    if (target_time_stride < 0) return RC_ERR_BAD_SHAPE;
    return interp_dispatch(&s, 1, &source_time_stride, target_times, target_time_stride, out, B, T, dtype, device, stream);
}

int rc_resample_ragged(const void* src_rows, const float* source_times, const int64_t* row_offsets, int64_t max_len,
                       const float* target_times, void* out, int64_t B, int64_t T, int64_t D, int dtype, int device,
                       void* stream) {
    return ragged_dispatch(src_rows, source_times, reinterpret_cast<const long long*>(row_offsets), max_len,
                           target_times, out, B, T, D, dtype, device, stream);
}

int rc_fuse(const rc_stream_desc* streams, int n_streams, const float* target_times, void* out,
            int64_t B, int64_t T, int dtype, int device, void* stream) {
    return interp_dispatch(streams, n_streams, nullptr, target_times, -1, out, B, T, dtype, device, stream);
}

int rc_fuse_strided(const rc_stream_desc* streams, const int64_t* time_strides, int n_streams, const float* target_times,
                    int64_t target_time_stride, void* out, int64_t B, int64_t T, int dtype, int device, void* stream) {
    if (time_strides == nullptr) return RC_ERR_NULL_POINTER;
    if (target_time_stride < 0) return RC_ERR_BAD_SHAPE;
    return interp_dispatch(streams, n_streams, time_strides, target_times, target_time_stride, out, B, T, dtype, device,
                           stream);
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

int rc_bulk_wait_timeouts(int device, unsigned int* count_host) {
    if (count_host == nullptr) return RC_ERR_NULL_POINTER;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    RC_CUDA_TRY(cudaMemcpyFromSymbol(count_host, g_bulk_wait_timeouts, sizeof(unsigned int)));
    return RC_OK;
}

}  // extern "C"
