// Bandwidth-bound helper kernels around the tensor-core pipeline: row gather/pad,
// correct-token gather-dot, log-sum-exp merge, column sums and the final cast/scatter.
#pragma once
#include <cooperative_groups.h>
#include "engine.cuh"

namespace cce {

__device__ __forceinline__ long long load_index(const void* idx, int is_i64, long long i) {
    return is_i64 ? reinterpret_cast<const long long*>(idx)[i]
                  : (long long)reinterpret_cast<const int*>(idx)[i];
}

// Row count of a launch: the host's value, or (when the caller kept the count on the device and
// sized the launch for an upper bound) min(*n_dev, bound).
__device__ __forceinline__ long long actual_rows(long long bound, const long long* n_dev) {
    if (!n_dev) return bound;
    const long long n = *n_dev;
    return n < 0 ? 0 : (n < bound ? n : bound);
}

__device__ __forceinline__ float load_as_float(const void* p, int dtype, long long i) {
    if (dtype == 2) return reinterpret_cast<const float*>(p)[i];
    if (dtype == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

// dst[i][0..Dp) = src[rows[i]][0..D) (16-bit elements), zero padded to Dp columns.
// One block per output row; rows past a device-side count (n_dev) are written as zeros.
__global__ void pack_rows_kernel(const uint16_t* __restrict__ src, long long ld_src,
                                 const void* __restrict__ rows, int rows_i64, uint16_t* __restrict__ dst,
                                 long long Dp, long long D, long long n_rows, const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x;
    if (i >= n_rows) return;
    uint16_t* d = dst + i * Dp;
    if (i >= actual_rows(n_rows, n_dev)) {  // past the list: a row of zeros
        for (long long j = threadIdx.x; j < Dp; j += blockDim.x) d[j] = 0;
        return;
    }
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const uint16_t* s = src + r * ld_src;
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

// fp32 operands run on the bf16 tensor path as a three-term split: x = hi + lo with hi = bf16(x),
// lo = bf16(x - hi), and  e.c ~= e_hi.c_hi + e_hi.c_lo + e_lo.c_hi  (error ~2^-16 relative).
// This kernel writes one staged row of 3*Dp bf16: pattern 0 (embeddings) = [hi | hi | lo],
// pattern 1 (classifier) = [hi | lo | hi], each block zero-padded from D to Dp columns, so that
// one K = 3*Dp contraction of the staged rows gives the three-term sum.  One block per row.
__global__ void split_rows_kernel(const float* __restrict__ src, long long ld_src, const void* __restrict__ rows,
                                  int rows_i64, __nv_bfloat16* __restrict__ dst, long long Dp, long long D,
                                  long long n_rows, int pattern, const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x;
    if (i >= n_rows) return;
    __nv_bfloat16* d = dst + i * 3 * Dp;
    if (i >= actual_rows(n_rows, n_dev)) {
        for (long long j = threadIdx.x; j < 3 * Dp; j += blockDim.x) d[j] = __float2bfloat16_rn(0.0f);
        return;
    }
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const float* s = src + r * ld_src;
    for (long long j = threadIdx.x; j < Dp; j += blockDim.x) {
        const float x = j < D ? s[j] : 0.0f;
        const __nv_bfloat16 hi = __float2bfloat16_rn(x);
        const __nv_bfloat16 lo = __float2bfloat16_rn(x - __bfloat162float(hi));
        d[j] = hi;
        d[Dp + j] = pattern == 0 ? hi : lo;
        d[2 * Dp + j] = pattern == 0 ? lo : hi;
    }
}

__global__ void to_f32_kernel(const void* __restrict__ src, int dtype, float* __restrict__ dst, long long n) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) dst[i] = load_as_float(src, dtype, i);
}

// lse[row] = ln2 * (M + log2(sum_b s_b * 2^(m_b - M))) over the bands of the forward kernel.
// A non-zero status word (a pipeline kernel abandoned a wait, so `partial` is incomplete) turns
// every output into NaN: the failure shows in the loss without a host read of the word.
__global__ void lse_combine_kernel(const float2* __restrict__ partial, int n_band, long long n_rows,
                                   float* __restrict__ lse, const int* __restrict__ status,
                                   const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= actual_rows(n_rows, n_dev)) return;  // `partial` keeps the pitch n_rows
    if (status && *status != 0) {
        lse[i] = __int_as_float(0x7fc00000);
        return;
    }
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
                                       int has_softcap, float softcap, float* __restrict__ out,
                                       const long long* __restrict__ n_dev) {
    const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i >= actual_rows(n_rows, n_dev)) return;
    const long long r = valids ? load_index(valids, valids_i64, i) : i;
    const long long t = targets[r + shift] - vocab_start;
    if (t < 0 || t >= V) {
        if (lane == 0) out[i] = 0.0f;
        return;
    }
    const T* ep = e + r * lde;
    const T* cp = c + t * ldc;
    float acc = 0.0f;
    constexpr int VE = 16 / int(sizeof(T));  // elements per 16-byte load
    const bool vec = (D % VE == 0) && ((reinterpret_cast<uintptr_t>(ep) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
    if (vec) {
        const uint4* e4 = reinterpret_cast<const uint4*>(ep);
        const uint4* c4 = reinterpret_cast<const uint4*>(cp);
        for (long long j = lane; j < D / VE; j += 32) {
            const uint4 a = __ldg(e4 + j), b = __ldg(c4 + j);
            const T* ah = reinterpret_cast<const T*>(&a);
            const T* bh = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int k = 0; k < VE; ++k) acc = fmaf(float(ah[k]), float(bh[k]), acc);
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
                                        float* __restrict__ out, int n_groups, const long long* __restrict__ n_dev) {
    const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (g >= n_groups) return;
    n_rows = actual_rows(n_rows, n_dev);  // groups past the count get +inf: nothing there is ever active
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
                                 uint8_t* __restrict__ act, const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < actual_rows(n_rows, n_dev)) {
        const long long r = valids ? load_index(valids, valids_i64, i) : i;
        const long long t = targets[r + shift] - vocab_start;
        if (t >= 0 && t < V) act[(i >> 7) * n_vt + (t >> 8)] = 1;
    }
    if (i < (long long)n_groups * n_vt) {
        const int g = int(i / n_vt), vt = int(i % n_vt);
        if (tile_max[i] - min_lse2[g] >= log2_eps) act[(size_t)(g >> 2) * n_vt + vt] = 1;
    }
}

// ---- vocabulary ordering (the classifier rows are visited in a caller-given order, so that the
// columns that hold large probabilities share few tiles)
// One block per 256 positions of the order: inv_order[order[i]] = i, and tile_colmax[T] = the largest
// column maximum (log2 units) among the 256 columns that make up reordered tile T.
__global__ void __launch_bounds__(256)
order_prepare_kernel(const int* __restrict__ order, long long V, const int* __restrict__ col_max_key,
                     int* __restrict__ inv_order, float* __restrict__ tile_colmax) {
    __shared__ int warp_max[8];
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    int k = INT_MIN;
    if (i < V) {
        const int o = order[i];
        inv_order[o] = int(i);
        k = col_max_key[o];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) k = max(k, __shfl_xor_sync(0xffffffffu, k, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = k;
    __syncthreads();
    if (threadIdx.x == 0) {
        int m = warp_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = max(m, warp_max[w]);
        tile_colmax[blockIdx.x] = key_to_float(m);
    }
}

// dst[i] = float(src[order[i]])
__global__ void gather_f32_kernel(const void* __restrict__ src, int dtype, const int* __restrict__ order,
                                  float* __restrict__ dst, long long n) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) dst[i] = load_as_float(src, dtype, order[i]);
}

// tile_mark_kernel for a reordered vocabulary.  Reordered tile T (columns order[256 T .. 256 T + 255])
// can hold a value >= eps for 32-row group g only if BOTH upper bounds of its softmax values allow it:
//   tile_colmax[T] - min_lse[g]                                   (column maxima over all rows)
//   max_j tile_max[g][order[256 T + j] / 256] - min_lse[g]        (the forward's per-tile maxima)
// One warp per (g, T) pair evaluates the second bound only where the first one passes.  Thread i < n_rows
// also marks the tile that holds row i's label (its position in the order comes from inv_order).
__global__ void tile_mark_ordered_kernel(const float* __restrict__ tile_max, const float* __restrict__ min_lse2,
                                         const float* __restrict__ tile_colmax, const int* __restrict__ order,
                                         const int* __restrict__ inv_order, int n_groups, int n_vt, float log2_eps,
                                         const long long* __restrict__ targets, const void* __restrict__ valids,
                                         int valids_i64, long long shift, long long vocab_start, long long V,
                                         long long n_rows, uint8_t* __restrict__ act,
                                         const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < actual_rows(n_rows, n_dev)) {
        const long long r = valids ? load_index(valids, valids_i64, i) : i;
        const long long t = targets[r + shift] - vocab_start;
        if (t >= 0 && t < V) act[(i >> 7) * n_vt + (inv_order[t] >> 8)] = 1;
    }
    const long long w = i >> 5;
    const int lane = threadIdx.x & 31;
    if (w < (long long)n_groups * n_vt) {
        const int g = int(w / n_vt), T = int(w % n_vt);
        const float floor2 = min_lse2[g] + log2_eps;
        if (tile_colmax[T] >= floor2) {  // warp-uniform
            float m = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const long long pos = (long long)T * 256 + j * 32 + lane;
                if (pos < V) m = fmaxf(m, tile_max[(size_t)g * n_vt + (order[pos] >> 8)]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0 && m >= floor2) act[(size_t)(g >> 2) * n_vt + T] = 1;
        }
    }
}

// ---- mean logit per vocabulary entry (the reference's ordering key, cce_lse_forward.py:95-97):
// logit_avg[v] = softcap(mean_rows(e) . c[v] + bias[v]).  Without soft-capping that is the mean of
// the logits of column v; with it, the soft-cap of the mean (monotone in it, hence the same order).
// Stage 1: partial[slice][d] = sum of the listed rows [slice * rows_per_block, ...) of column d.
template <typename T>
__global__ void rows_colsum_partial_kernel(const T* __restrict__ e, long long lde, const void* __restrict__ valids,
                                           int valids_i64, long long n_rows, long long D, int rows_per_block,
                                           float* __restrict__ partial, const long long* __restrict__ n_dev) {
    const long long d = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    n_rows = actual_rows(n_rows, n_dev);
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(n_rows, r0 + rows_per_block);
    float s = 0.0f;
    for (long long i = r0; i < r1; ++i) {
        const long long r = valids ? load_index(valids, valids_i64, i) : i;
        s += float(e[r * lde + d]);
    }
    partial[(size_t)blockIdx.y * D + d] = s;
}
// Stage 2: mean_e[d] = (sum over the slices, ascending) / n_rows
__global__ void rows_colsum_finish_kernel(const float* __restrict__ partial, int n_slices, long long D,
                                          long long n_rows, float* __restrict__ mean_e,
                                          const long long* __restrict__ n_dev) {
    const long long d = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    n_rows = actual_rows(n_rows, n_dev);
    float s = 0.0f;
    for (int k = 0; k < n_slices; ++k) s += partial[(size_t)k * D + d];
    mean_e[d] = s / float(n_rows > 0 ? n_rows : 1);
}
// Stage 3: one warp per vocabulary entry
template <typename T>
__global__ void logit_avg_kernel(const float* __restrict__ mean_e, const T* __restrict__ c, long long ldc,
                                 const void* __restrict__ bias, int bias_dtype, long long V, long long D,
                                 int has_softcap, float softcap, float* __restrict__ out) {
    const long long v = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (v >= V) return;
    const T* cp = c + v * ldc;
    float acc = 0.0f;
    constexpr int VE = 16 / int(sizeof(T));
    const bool vec = (D % VE == 0) && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
    if (vec) {
        const uint4* c4 = reinterpret_cast<const uint4*>(cp);
        for (long long j = lane; j < D / VE; j += 32) {
            const uint4 b = __ldg(c4 + j);
            const T* bh = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int k = 0; k < VE; ++k) acc = fmaf(__ldg(mean_e + j * VE + k), float(bh[k]), acc);
        }
    } else {
        for (long long j = lane; j < D; j += 32) acc = fmaf(mean_e[j], float(cp[j]), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        if (bias) acc += load_as_float(bias, bias_dtype, v);
        if (has_softcap) acc = softcap * tanhf(acc / softcap);
        out[v] = acc;
    }
}

// Index of the active tiles (one block of 1024 threads; dynamic smem = (n_vt + n_rb + 2) ints).
// Slots number the active tiles column by column (vt ascending, then rb), so column vt owns the
// contiguous slots [col_ptr[vt], col_ptr[vt+1]); row_slots lists each row block's slots with vt
// ascending (CSR).  Passes split the columns greedily so that each pass holds at most `capacity`
// slots: pass_info[4p..4p+3] = {vt_lo, vt_hi, slot_lo, slot_hi}; unused passes are empty.
__global__ void tile_index_kernel(const uint8_t* __restrict__ act, int n_rb, int n_vt, int capacity,
                                  int max_pass, int* __restrict__ col_ptr, int* __restrict__ slot_tile,
                                  int* __restrict__ slot_of, int* __restrict__ row_ptr,
                                  int* __restrict__ row_slots, int* __restrict__ pass_info,
                                  int* __restrict__ counts_out, long long n_rows, const long long* __restrict__ n_dev) {
    extern __shared__ int sm[];
    int* col_s = sm;              // [n_vt + 1] column counts, then column starts
    int* row_s = sm + n_vt + 1;   // [n_rb + 1] row counts, then row starts
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
    for (int rb = tid; rb < n_rb; rb += nthr) row_s[rb] = 0;
    __syncthreads();
    // per-column counts (thread per column; neighbouring threads read neighbouring bytes)
    for (int vt = tid; vt < n_vt; vt += nthr) {
        int cnt = 0;
        for (int rb0 = 0; rb0 < n_rb; rb0 += 8) {  // 8 independent loads in flight per step
            uint8_t v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (rb0 + j < n_rb) ? act[(size_t)(rb0 + j) * n_vt + vt] : 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (v[j]) {
                    ++cnt;
                    atomicAdd(&row_s[rb0 + j], 1);
                }
            }
        }
        col_s[vt] = cnt;
    }
    __syncthreads();
    {   // column starts: exclusive scan of the counts, a contiguous run of columns per thread
        __shared__ int warp_sum[32];
        const int per = (n_vt + nthr - 1) / nthr;
        const int beg = min(tid * per, n_vt), end = min(beg + per, n_vt);
        int local = 0;
        for (int vt = beg; vt < end; ++vt) local += col_s[vt];
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int v = lane < nwarp ? warp_sum[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            warp_sum[lane] = v;
        }
        __syncthreads();
        int run = incl - local + (warp > 0 ? warp_sum[warp - 1] : 0);
        for (int vt = beg; vt < end; ++vt) {
            const int cnt = col_s[vt];
            col_s[vt] = run;
            col_ptr[vt] = run;
            run += cnt;
        }
        if (tid == nthr - 1) {
            col_s[n_vt] = warp_sum[nwarp - 1];
            col_ptr[n_vt] = warp_sum[nwarp - 1];
        }
    }
    __syncthreads();
    if (tid == 0) {  // pass boundaries: each pass takes whole columns while it holds <= capacity slots
        const int total = col_s[n_vt];
        int pass = 0, vt0 = 0;
        while (true) {
            const int s0 = col_s[vt0];
            int vt_end = n_vt;
            if (pass + 1 < max_pass && total - s0 > capacity) {
                int lo = vt0 + 1, hi = n_vt;  // largest v in [lo, hi] with col_s[v] - s0 <= capacity
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (col_s[mid] - s0 <= capacity) lo = mid; else hi = mid - 1;
                }
                vt_end = lo;
            }
            pass_info[4 * pass + 0] = vt0;
            pass_info[4 * pass + 1] = vt_end;
            pass_info[4 * pass + 2] = s0;
            pass_info[4 * pass + 3] = col_s[vt_end];
            if (vt_end == n_vt) break;
            ++pass;
            vt0 = vt_end;
        }
        if (counts_out) {  // optional report: {active tiles, all tiles, passes that hold tiles}
            counts_out[0] = total;
            counts_out[1] = int((actual_rows(n_rows, n_dev) + 127) / 128) * n_vt;  // row blocks that hold rows
            counts_out[2] = total > 0 ? pass + 1 : 0;
        }
        for (int q = pass + 1; q < max_pass; ++q) {
            pass_info[4 * q + 0] = n_vt;
            pass_info[4 * q + 1] = n_vt;
            pass_info[4 * q + 2] = total;
            pass_info[4 * q + 3] = total;
        }
    } else if (tid == 32) {  // row starts
        int run = 0;
        for (int rb = 0; rb < n_rb; ++rb) {
            const int cnt = row_s[rb];
            row_ptr[rb] = run;
            row_s[rb] = run;
            run += cnt;
        }
        row_ptr[n_rb] = run;
    }
    __syncthreads();
    // slots, column by column
    for (int vt = tid; vt < n_vt; vt += nthr) {
        int k = col_s[vt];
        for (int rb0 = 0; rb0 < n_rb; rb0 += 8) {
            uint8_t v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (rb0 + j < n_rb) ? act[(size_t)(rb0 + j) * n_vt + vt] : 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (v[j]) {
                    slot_tile[k] = (rb0 + j) * n_vt + vt;
                    slot_of[(size_t)(rb0 + j) * n_vt + vt] = k;
                    ++k;
                }
            }
        }
    }
    __syncthreads();
    // row lists (one warp per row block, 128 columns per step, order kept by an in-warp scan)
    for (int rb = warp; rb < n_rb; rb += nwarp) {
        int k = row_s[rb];
        for (int v0 = 0; v0 < n_vt; v0 += 128) {
            uint32_t bits = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int vt = v0 + lane * 4 + j;
                if (vt < n_vt && act[(size_t)rb * n_vt + vt]) bits |= 1u << j;
            }
            const int c = __popc(bits);
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            int pos = k + incl - c;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (bits & (1u << j)) row_slots[pos++] = slot_of[(size_t)rb * n_vt + v0 + lane * 4 + j];
            k += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
}

// After phase 1 of a pass: turn the slot flags into ordered K-block lists for the two products
// (one warp per list), clearing every flag it reads so that the next pass starts from zeros.  Warps 0..n_rb-1 build the dE list of a row block: its slots that belong to
// the pass, vt ascending, 4 column groups each.  The next 2*n_vt warps build the dC list of a
// (vt, 128-column half): its slots, rb ascending, 2 row halves each.  Layout: see EngineParams.
__global__ void klist_build_kernel(const int* __restrict__ pass_info, const int* __restrict__ row_ptr,
                                   const int* __restrict__ row_slots, const int* __restrict__ col_ptr,
                                   const int* __restrict__ slot_tile, int n_rb, int n_vt,
                                   uint8_t* __restrict__ sflag_e, uint8_t* __restrict__ sflag_c,
                                   int2* __restrict__ de_list, int* __restrict__ de_cnt,
                                   int2* __restrict__ dc_list, int* __restrict__ dc_cnt) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int vt_lo = pass_info[0], vt_hi = pass_info[1], s_lo = pass_info[2], s_hi = pass_info[3];
    if (s_lo == s_hi) {  // an empty pass: every list is empty
        if (lane == 0 && w < n_rb) de_cnt[w] = 0;
        if (lane == 0 && w >= n_rb && w < n_rb + 2 * n_vt) dc_cnt[w - n_rb] = 0;
        return;
    }
    if (w < n_rb) {
        const int e0 = row_ptr[w], n = (row_ptr[w + 1] - e0) * 4;
        int2* out = de_list + 4 * e0;
        int k = 0;
        for (int c0 = 0; c0 < n; c0 += 32) {
            const int c = c0 + lane;
            bool on = false;
            int2 ent = make_int2(0, 0);
            if (c < n) {
                const int slot = row_slots[e0 + (c >> 2)];
                if (slot >= s_lo && slot < s_hi) {
                    const int sl = slot - s_lo, kb = c & 3;
                    on = sflag_e[sl * 4 + kb] != 0;
                    if (on) sflag_e[sl * 4 + kb] = 0;  // each flag has one reader: leave it clear for the next pass
                    ent = make_int2(sl * 4 + kb, slot_tile[slot] % n_vt);
                }
            }
            const uint32_t m = __ballot_sync(0xffffffffu, on);
            if (on) out[k + __popc(m & ((1u << lane) - 1u))] = ent;
            k += __popc(m);
        }
        if (lane == 0) de_cnt[w] = k;
    } else if (w < n_rb + 2 * n_vt) {
        const int id = w - n_rb, vt = id >> 1, h = id & 1;
        int k = 0;
        if (vt >= vt_lo && vt < vt_hi) {
            const int c0s = col_ptr[vt], ns = col_ptr[vt + 1] - c0s, n = ns * 2;
            int2* out = dc_list + 4 * c0s + 2 * h * ns;
            for (int c0 = 0; c0 < n; c0 += 32) {
                const int c = c0 + lane;
                bool on = false;
                int2 ent = make_int2(0, 0);
                if (c < n) {
                    const int slot = c0s + (c >> 1), sl = slot - s_lo, kb = c & 1;
                    on = sflag_c[sl * 4 + h * 2 + kb] != 0;
                    if (on) sflag_c[sl * 4 + h * 2 + kb] = 0;
                    ent = make_int2(sl * 2 + kb, slot_tile[slot] / n_vt);
                }
                const uint32_t m = __ballot_sync(0xffffffffu, on);
                if (on) out[k + __popc(m & ((1u << lane) - 1u))] = ent;
                k += __popc(m);
            }
        }
        if (lane == 0) dc_cnt[id] = k;
    }
}

// Column sums of a [n_rows][width] 16-bit block with pitch ldg, in two deterministic stages.
// Stage 1: partial[rb][col] = sum of rows [rb * rows_per_block, (rb + 1) * rows_per_block) of column col;
// grid = (ceil(width/256), ceil(n_rows/rows_per_block)); 128 threads, two columns each.
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ g, long long ldg, long long n_rows, int width,
                                      int rows_per_block, float* __restrict__ partial, long long ld_partial,
                                      const long long* __restrict__ n_dev) {
    const int col = (blockIdx.x * 128 + threadIdx.x) * 2;
    if (col >= width) return;
    n_rows = actual_rows(n_rows, n_dev);  // a slice past the count sums nothing and writes 0
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(n_rows, r0 + rows_per_block);
    float* out = partial + (size_t)blockIdx.y * ld_partial + col;
    float s0 = 0.0f, s1 = 0.0f;
    if (col + 1 < width) {
        for (long long r = r0; r < r1; ++r) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(g + r * ldg + col);
            const T* h = reinterpret_cast<const T*>(&w);
            s0 += float(h[0]);
            s1 += float(h[1]);
        }
        out[0] = s0;
        out[1] = s1;
    } else {
        for (long long r = r0; r < r1; ++r) s0 += float(g[r * ldg + col]);
        out[0] = s0;
    }
}
// Stage 2: dbias[col] = sum over the row blocks, in ascending order (no atomics: the same bits every run).
__global__ void colsum_finish_kernel(const float* __restrict__ partial, long long ld_partial, int n_rowblk,
                                     int width, float* __restrict__ dbias) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= width) return;
    float s = 0.0f;
    for (int rb = 0; rb < n_rowblk; ++rb) s += partial[(size_t)rb * ld_partial + col];
    dbias[col] = s;
}

// A non-zero status word (a pipeline kernel abandoned a wait) turns the rows into NaN.
template <typename T>
__global__ void scatter_cast_kernel(const float* __restrict__ src, long long ld_src,
                                    const void* __restrict__ rows, int rows_i64, T* __restrict__ dst,
                                    long long ld_dst, long long D, long long n_rows,
                                    const int* __restrict__ status, const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x;
    if (i >= actual_rows(n_rows, n_dev)) return;
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const float* s = src + i * ld_src;
    T* d = dst + r * ld_dst;
    const bool bad = status && *status != 0;
    const bool vec = !bad && (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(s) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(d) & (4 * sizeof(T) - 1)) == 0);
    if (vec) {
        for (long long j = threadIdx.x; j < D / 4; j += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(s)[j];
            if constexpr (sizeof(T) == 4) {
                reinterpret_cast<float4*>(d)[j] = v;
            } else {
                T o[4] = {T(v.x), T(v.y), T(v.z), T(v.w)};
                reinterpret_cast<uint2*>(d)[j] = *reinterpret_cast<const uint2*>(o);
            }
        }
    } else {
        for (long long j = threadIdx.x; j < D; j += blockDim.x) d[j] = bad ? T(__int_as_float(0x7fc00000)) : T(s[j]);
    }
}

// dE summed across ranks by the product kernels themselves (EngineParams::peer_world): this rank's
// accumulator `acc` [acc_rows][D] fp32 holds the finished sums of the row blocks it owns.  Writes
// them to `slice` in the output type and clears the accumulator for the next step.  A non-zero
// status word (one of this rank's kernels abandoned a wait, so its contributions are missing
// everywhere) turns the slice into NaN, which the exchange that follows carries to every rank.
template <typename T>
__global__ void peer_collect_kernel(float* __restrict__ acc, long long n, T* __restrict__ slice,
                                    const int* __restrict__ status) {
    const bool bad = status && *status != 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n / 4; i += stride) {
        float4 v = reinterpret_cast<float4*>(acc)[i];
        reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bad) v.x = v.y = v.z = v.w = __int_as_float(0x7fc00000);
        if constexpr (sizeof(T) == 4) {
            reinterpret_cast<float4*>(slice)[i] = v;
        } else {
            T o[4] = {T(v.x), T(v.y), T(v.z), T(v.w)};
            reinterpret_cast<uint2*>(slice)[i] = *reinterpret_cast<const uint2*>(o);
        }
    }
}

// peer_collect_kernel with the exchange built in: the cast rows go straight to slot `rank` of every
// rank's gather buffer [world][n] (mapped peer memory, 16-byte stores), so that no collective has to
// move them afterwards.  n is a multiple of 8.
struct PeerPtrs {
    void* p[kMaxPeers];
};
template <typename T>
__global__ void peer_collect_push_kernel(float* __restrict__ acc, long long n, PeerPtrs gath, int world, int rank,
                                         const int* __restrict__ status) {
    const bool bad = status && *status != 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    constexpr int PER = 16 / sizeof(T);  // values per 16-byte store: 8 (16-bit) or 4 (fp32)
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n / PER; i += stride) {
        float v[PER];
#pragma unroll
        for (int j = 0; j < PER / 4; ++j) {
            const float4 x = reinterpret_cast<float4*>(acc)[i * (PER / 4) + j];
            reinterpret_cast<float4*>(acc)[i * (PER / 4) + j] = make_float4(0.f, 0.f, 0.f, 0.f);
            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
        }
        if (bad) {
#pragma unroll
            for (int j = 0; j < PER; ++j) v[j] = __int_as_float(0x7fc00000);
        }
        uint4 out;
        if constexpr (sizeof(T) == 4) {
            out = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
        } else {
            T o[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) o[j] = T(v[j]);
            out = *reinterpret_cast<const uint4*>(o);
        }
        for (int r = 0; r < world; ++r) {
            const int dst = (rank + 1 + r) % world;  // ranks start at different peers; the own copy goes last
            reinterpret_cast<uint4*>(reinterpret_cast<T*>(gath.p[dst]) + (long long)rank * n)[i] = out;
        }
    }
}

// The gathered slices [world][acc_rows][D] back to the caller's rows: packed row i belongs to row
// block m = i / 128, owned by rank m % world at rows (m / world) * 128 + i % 128 of its slice.
template <typename T>
__global__ void peer_scatter_kernel(const T* __restrict__ gathered, int world, long long acc_rows, long long D,
                                    const void* __restrict__ rows, int rows_i64, T* __restrict__ dst,
                                    long long n_rows, const long long* __restrict__ n_dev) {
    const long long i = blockIdx.x;
    if (i >= actual_rows(n_rows, n_dev)) return;
    const long long r = rows ? load_index(rows, rows_i64, i) : i;
    const long long m = i / 128;
    const T* s = gathered + ((m % world) * acc_rows + (m / world) * 128 + (i % 128)) * D;
    T* d = dst + r * D;
    constexpr int VEC = 16 / sizeof(T);
    if (D % VEC == 0 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
        for (long long j = threadIdx.x; j < D / VEC; j += blockDim.x)
            reinterpret_cast<uint4*>(d)[j] = reinterpret_cast<const uint4*>(s)[j];
    } else {
        for (long long j = threadIdx.x; j < D; j += blockDim.x) d[j] = s[j];
    }
}

// Tail of the forward pass in one block: merges the per-rank statistics, forms the negative
// log-likelihood of every row and reduces or scatters it.
//   stats[r][0][i] = log-sum-exp of row i over rank r's vocabulary shard, stats[r][1][i] = minus the
//   correct-token logit (0 on ranks that do not own the label); `world` ranks, rank pitch 2 * n_rows.
//   lse_i = logsumexp_r stats[r][0][i],  nll_i = lse_i + sum_r stats[r][1][i]
//   reduction 0 / 1: loss_out[0] = mean / sum of nll (fixed summation order: deterministic)
//   reduction 2    : loss_out[pos_i] = nll_i, pos_i = rows[i] + shift (rows null: i)
//   lse_rows (optional) [n_rows] receives lse_i; lse_scatter (optional) receives lse_i at pos_i.
// Positions that no row maps to are cleared by the caller before the launch.
constexpr int TAIL_THREADS = 1024;
constexpr int TAIL_CTAS = 8;  // one cluster; rows are dealt to its CTAs 1024 at a time
__global__ void __cluster_dims__(TAIL_CTAS, 1, 1) __launch_bounds__(TAIL_THREADS)
loss_tail_kernel(const float* __restrict__ stats, int world, long long n_rows, const void* __restrict__ rows,
                 int rows_i64, long long shift, int reduction, float* __restrict__ lse_rows,
                 float* __restrict__ loss_out, float* __restrict__ lse_scatter, const int* __restrict__ status,
                 const long long* __restrict__ n_dev) {
    __shared__ double warp_sum[TAIL_THREADS / 32];
    __shared__ double cta_sum;
    const bool bad = status && *status != 0;
    double acc = 0.0;
    const long long n_act = actual_rows(n_rows, n_dev);  // `stats` keeps the pitch n_rows
    for (long long i = (long long)blockIdx.x * TAIL_THREADS + threadIdx.x; i < n_act; i += TAIL_CTAS * TAIL_THREADS) {
        float m = -INFINITY, neg = 0.0f;
        for (int r = 0; r < world; ++r) {
            m = fmaxf(m, stats[(size_t)r * 2 * n_rows + i]);
            neg += stats[((size_t)r * 2 + 1) * n_rows + i];
        }
        float lse = m;
        if (world > 1 && m > -INFINITY) {
            float ssum = 0.0f;
            for (int r = 0; r < world; ++r) ssum += expf(stats[(size_t)r * 2 * n_rows + i] - m);
            lse = m + logf(ssum);
        }
        float nll = lse + neg;
        if (bad) lse = nll = __int_as_float(0x7fc00000);
        const long long pos = rows ? load_index(rows, rows_i64, i) + shift : i;
        if (lse_rows) lse_rows[i] = lse;
        if (lse_scatter) lse_scatter[pos] = lse;
        if (reduction == 2) loss_out[pos] = nll;
        acc += (double)nll;
    }
    if (reduction == 2) return;  // uniform over the cluster
    // fixed summation order (lanes, warps, CTAs): the same inputs always give the same bits
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < TAIL_THREADS / 32; ++w) t += warp_sum[w];
        cta_sum = t;
    }
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    cluster.sync();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        double t = 0.0;
        for (int r = 0; r < TAIL_CTAS; ++r) t += *cluster.map_shared_rank(&cta_sum, r);
        loss_out[0] = float(reduction == 0 ? t / double(n_act) : t);
    }
    cluster.sync();  // no CTA leaves while its sum may still be read
}

// One warp waits on an mbarrier at which nobody ever arrives, with a caller-chosen cycle limit: the
// wait gives up, the status word receives ERR_WAIT_TMEM_FULL and the kernel returns normally.  It
// exercises the bounded-wait path of the pipeline kernels (mbar_wait) without touching TMA, tensor
// memory or the tensor cores.
__global__ void selftest_wait_kernel(long long limit_cycles, int* __restrict__ status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    // every lane waits, as the epilogue warps of the pipeline do; the first to time out raises the
    // abort flag, the others see it at their next poll
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, ERR_WAIT_TMEM_FULL, limit_cycles);
}

// ---- rows that enter the loss (ordered stream compaction in two launches)
// Row r of the flattened embeddings is paired with label targets[r + shift]; it is valid when the
// label lies in the same sequence (r % seq_len < seq_len - shift) and differs from ignore_index.
constexpr int VR_THREADS = 256;
constexpr int VR_PER_THREAD = 8;
constexpr int VR_BLOCK = VR_THREADS * VR_PER_THREAD;

__device__ __forceinline__ uint32_t valid_row_bits(const long long* __restrict__ targets, long long n_total,
                                                   long long seq_len, long long shift, long long ignore_index,
                                                   long long r0) {
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < VR_PER_THREAD; ++j) {
        const long long r = r0 + j;
        if (r < n_total && (shift == 0 || r % seq_len < seq_len - shift) && targets[r + shift] != ignore_index)
            bits |= 1u << j;
    }
    return bits;
}

// Sum over the block of one int per thread (VR_THREADS threads); every thread gets the total and
// its own exclusive prefix.
__device__ __forceinline__ int block_scan_256(int v, int* total) {
    __shared__ int warp_tot[VR_THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();  // the previous use of warp_tot is over
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < VR_THREADS / 32; ++w) {
        const int t = warp_tot[w];
        if (w < warp) before += t;
        all += t;
    }
    *total = all;
    return before + incl - v;
}

__global__ void set_count_kernel(long long* __restrict__ count_out, long long v) { count_out[0] = v; }

// block_counts[b] = valid rows among rows [b * VR_BLOCK, (b + 1) * VR_BLOCK)
__global__ void __launch_bounds__(VR_THREADS)
valid_rows_count_kernel(const long long* __restrict__ targets, long long n_total, long long seq_len,
                        long long shift, long long ignore_index, int* __restrict__ block_counts) {
    const long long r0 = (long long)blockIdx.x * VR_BLOCK + threadIdx.x * VR_PER_THREAD;
    int total;
    block_scan_256(__popc(valid_row_bits(targets, n_total, seq_len, shift, ignore_index, r0)), &total);
    if (threadIdx.x == 0) block_counts[blockIdx.x] = total;
}

// rows_out[k] = k-th valid row (ascending), as int32 or int64; count_out[0] = number of valid rows
__global__ void __launch_bounds__(VR_THREADS)
valid_rows_write_kernel(const long long* __restrict__ targets, long long n_total, long long seq_len,
                        long long shift, long long ignore_index, const int* __restrict__ block_counts,
                        void* __restrict__ rows_out, int rows_i64, long long* __restrict__ count_out) {
    int before = 0;  // valid rows of the blocks before this one
    for (int b = threadIdx.x; b < (int)blockIdx.x; b += VR_THREADS) before += block_counts[b];
    int base;
    block_scan_256(before, &base);
    const long long r0 = (long long)blockIdx.x * VR_BLOCK + threadIdx.x * VR_PER_THREAD;
    const uint32_t bits = valid_row_bits(targets, n_total, seq_len, shift, ignore_index, r0);
    int total;
    long long k = (long long)base + block_scan_256(__popc(bits), &total);
#pragma unroll
    for (int j = 0; j < VR_PER_THREAD; ++j) {
        if (bits & (1u << j)) {
            if (rows_i64) reinterpret_cast<long long*>(rows_out)[k] = r0 + j;
            else reinterpret_cast<int*>(rows_out)[k] = int(r0 + j);
            ++k;
        }
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) count_out[0] = (long long)base + total;
}

}  // namespace cce
