// Bandwidth-bound helper kernels around the tensor-core pipeline: row gather/pad,
// correct-token gather-dot, log-sum-exp merge, column sums and the final cast/scatter.
#pragma once
#include "ptx.cuh"

namespace cce {

__device__ __forceinline__ long long load_index(const void* idx, int is_i64, long long i) {
    return is_i64 ? reinterpret_cast<const long long*>(idx)[i]
                  : (long long)reinterpret_cast<const int*>(idx)[i];
}

__device__ __forceinline__ float load_as_float(const void* p, int dtype, long long i) {
    if (dtype == 2) return reinterpret_cast<const float*>(p)[i];
    if (dtype == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

// dst[i][0..Dp) = src[rows[i]][0..D) (16-bit elements), zero padded to Dp columns.
// One block per output row.
__global__ void pack_rows_kernel(const uint16_t* __restrict__ src, long long ld_src,
                                 const void* __restrict__ rows, int rows_i64, uint16_t* __restrict__ dst,
                                 long long Dp, long long D, long long n_rows) {
    const long long i = blockIdx.x;
    if (i >= n_rows) return;
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const uint16_t* s = src + r * ld_src;
    uint16_t* d = dst + i * Dp;
    const bool vec = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && (D % 8 == 0);
    if (vec) {
        const uint4* s4 = reinterpret_cast<const uint4*>(s);
        uint4* d4 = reinterpret_cast<uint4*>(d);
        for (long long j = threadIdx.x; j < D / 8; j += blockDim.x) d4[j] = s4[j];
    } else {
        for (long long j = threadIdx.x; j < D; j += blockDim.x) d[j] = s[j];
    }
    for (long long j = D + threadIdx.x; j < Dp; j += blockDim.x) d[j] = 0;
}

__global__ void to_f32_kernel(const void* __restrict__ src, int dtype, float* __restrict__ dst, long long n) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) dst[i] = load_as_float(src, dtype, i);
}

// lse[row] = ln2 * (M + log2(sum_b s_b * 2^(m_b - M))) over the bands of the forward kernel.
__global__ void lse_combine_kernel(const float2* __restrict__ partial, int n_band, long long n_rows,
                                   float* __restrict__ lse) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= n_rows) return;
    float m = -INFINITY;
    for (int b = 0; b < n_band; ++b) m = fmaxf(m, partial[(size_t)b * n_rows + i].x);
    float s = 0.0f;
    if (m > -INFINITY) {
        for (int b = 0; b < n_band; ++b) {
            const float2 v = partial[(size_t)b * n_rows + i];
            s += v.y * exp2f(v.x - m);
        }
    }
    lse[i] = (m > -INFINITY) ? (m + log2f(s)) * kLn2 : -INFINITY;
}

// out[i] = -softcap(e[row_i] . c[t_i] + bias[t_i]); one warp per row, 16-byte loads when possible.
template <typename T>
__global__ void indexed_neg_dot_kernel(const T* __restrict__ e, long long lde, const T* __restrict__ c,
                                       long long ldc, const void* __restrict__ bias, int bias_dtype,
                                       const void* __restrict__ valids, int valids_i64,
                                       const long long* __restrict__ targets, long long shift,
                                       long long vocab_start, long long V, long long D, long long n_rows,
                                       int has_softcap, float softcap, float* __restrict__ out) {
    const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const long long r = valids ? load_index(valids, valids_i64, i) : i;
    const long long t = targets[r + shift] - vocab_start;
    if (t < 0 || t >= V) {
        if (lane == 0) out[i] = 0.0f;
        return;
    }
    const T* ep = e + r * lde;
    const T* cp = c + t * ldc;
    float acc = 0.0f;
    const bool vec = (D % 8 == 0) && ((reinterpret_cast<uintptr_t>(ep) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
    if (vec) {
        const uint4* e4 = reinterpret_cast<const uint4*>(ep);
        const uint4* c4 = reinterpret_cast<const uint4*>(cp);
        for (long long j = lane; j < D / 8; j += 32) {
            const uint4 a = __ldg(e4 + j), b = __ldg(c4 + j);
            const T* ah = reinterpret_cast<const T*>(&a);
            const T* bh = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc = fmaf(float(ah[k]), float(bh[k]), acc);
        }
    } else {
        for (long long j = lane; j < D; j += 32) acc = fmaf(float(ep[j]), float(cp[j]), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        if (bias) acc += load_as_float(bias, bias_dtype, t);
        if (has_softcap) acc = softcap * tanhf(acc / softcap);
        out[i] = -acc;
    }
}

// out[g] = log2(e) * min(lse[32g .. 32g+31]); one warp per group of 32 rows.
__global__ void rowgroup_min_lse_kernel(const float* __restrict__ lse, long long n_rows,
                                        float* __restrict__ out, int n_groups) {
    const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (g >= n_groups) return;
    const long long r = (long long)g * 32 + lane;
    float v = r < n_rows ? lse[r] * kLog2e : INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) out[g] = v;
}

// Marks the (128-row block, 256-column tile) pairs of the logit-gradient matrix that can hold an
// entry with |softmax - onehot| >= eps:  act[rb][vt] = 1 if the tile holds a label of one of its
// rows, or if for one of its four 32-row groups  tile_max - min_lse >= log2(eps)  (an upper
// bound of every softmax value in the group).  Thread i handles row i (labels) and pair i (bound).
__global__ void tile_mark_kernel(const float* __restrict__ tile_max, const float* __restrict__ min_lse2,
                                 int n_groups, int n_vt, float log2_eps, const long long* __restrict__ targets,
                                 const void* __restrict__ valids, int valids_i64, long long shift,
                                 long long vocab_start, long long V, long long n_rows,
                                 uint8_t* __restrict__ act) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n_rows) {
        const long long r = valids ? load_index(valids, valids_i64, i) : i;
        const long long t = targets[r + shift] - vocab_start;
        if (t >= 0 && t < V) act[(i >> 7) * n_vt + (t >> 8)] = 1;
    }
    if (i < (long long)n_groups * n_vt) {
        const int g = int(i / n_vt), vt = int(i % n_vt);
        if (tile_max[i] - min_lse2[g] >= log2_eps) act[(size_t)(g >> 2) * n_vt + vt] = 1;
    }
}

// Per vocabulary chunk, the compact list of active tiles: id = rb * tiles_per_chunk + tile-in-chunk.
// Thread index runs vocabulary-tile-major so that neighbours in a list share classifier tiles.
__global__ void tile_compact_kernel(const uint8_t* __restrict__ act, int n_rb, int n_vt, int tiles_per_chunk,
                                    int* __restrict__ lists, int* __restrict__ counts) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)n_rb * n_vt) return;
    const int vt = int(i / n_rb), rb = int(i % n_rb);
    if (!act[(size_t)rb * n_vt + vt]) return;
    const int ch = vt / tiles_per_chunk;
    const int slot = atomicAdd(counts + ch, 1);
    lists[(size_t)ch * n_rb * tiles_per_chunk + slot] = rb * tiles_per_chunk + (vt - ch * tiles_per_chunk);
}

// dbias[col] += sum_rows G[row][col] for a [n_rows][width] 16-bit block with pitch ldg.
// grid = (ceil(width/256), ceil(n_rows/rows_per_block)); 128 threads, two columns each.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ g, long long ldg, long long n_rows, int width,
                              int rows_per_block, float* __restrict__ dbias) {
    const int col = (blockIdx.x * 128 + threadIdx.x) * 2;
    if (col >= width) return;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(n_rows, r0 + rows_per_block);
    float s0 = 0.0f, s1 = 0.0f;
    if (col + 1 < width) {
        for (long long r = r0; r < r1; ++r) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(g + r * ldg + col);
            const T* h = reinterpret_cast<const T*>(&w);
            s0 += float(h[0]);
            s1 += float(h[1]);
        }
        atomicAdd(dbias + col, s0);
        atomicAdd(dbias + col + 1, s1);
    } else {
        for (long long r = r0; r < r1; ++r) s0 += float(g[r * ldg + col]);
        atomicAdd(dbias + col, s0);
    }
}

// d_e[rows[i]][0..D) = cast(src[i][0..D)); one block per row.
template <typename T>
__global__ void scatter_cast_kernel(const float* __restrict__ src, long long ld_src,
                                    const void* __restrict__ rows, int rows_i64, T* __restrict__ dst,
                                    long long ld_dst, long long D, long long n_rows) {
    const long long i = blockIdx.x;
    if (i >= n_rows) return;
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const float* s = src + i * ld_src;
    T* d = dst + r * ld_dst;
    for (long long j = threadIdx.x; j < D; j += blockDim.x) d[j] = T(s[j]);
}

}  // namespace cce
