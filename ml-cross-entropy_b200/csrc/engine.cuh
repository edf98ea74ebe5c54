// Persistent, warp-specialised TMA + tcgen05 contraction pipeline with three epilogues.
//
//   warp 0      : TMA producer  (global -> 128B-swizzled shared-memory ring)
//   warp 1      : tcgen05.mma issuer, owns the TMEM allocation (2 accumulators of 128x256 fp32)
//   warps 2..5  : epilogue; warp w reads TMEM lanes 32*(w%4)..+31, one output row per thread
//
// MODE_LSE   : S = E * C^T (+bias, softcap) -> running (max, sum-exp) per row over a band of
//              vocabulary tiles -> partial[band][row]                 (forward log-sum-exp)
// MODE_PGRAD : S recomputed -> G = dLoss/dS in bf16/fp16 -> G[row][col] plus per-block
//              "has a value >= eps" flags                             (backward, phase 1)
// MODE_GEMM  : out (+)= A * B over K with optional per-(row block, K block) skip flags
//              (backward, phases 2 and 3: dC = G^T E, dE += G C)
#pragma once
#include "ptx.cuh"

namespace cce {

constexpr int BM = 128;  // rows of the A side per tile  (TMEM lanes)
constexpr int BN = 256;  // rows of the B side per tile  (TMEM columns)
constexpr int BK = 64;   // reduction elements per stage (one 128-byte swizzle row of 16-bit data)
constexpr int UMMA_K = 16;
constexpr int NSTAGE = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ATOM_BYTES = 64 * 128;  // one MN-major swizzle atom column: 64 K rows x 128 bytes
constexpr int ENGINE_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int ENGINE_SMEM = NSTAGE * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
// Staging for the epilogue's bulk adds into peer memory (EngineParams::peer_world): one row of 32
// fp32 values per epilogue thread; the 144-byte pitch keeps the 16-byte stores of neighbouring
// threads in different banks.  Requested only by launches that add into peers.
constexpr int PEER_ROW_PITCH = 144;
constexpr int PEER_STAGE_BYTES = 4 * 32 * PEER_ROW_PITCH;

enum { MODE_LSE = 0, MODE_PGRAD = 1, MODE_GEMM = 2 };

// Wait-cycle tracing (EngineParams::wait_cycles) is compiled in only with -DCCE_TRACE=1: even
// switched off at run time its clock reads cost the forward kernel ~8 %.
#ifndef CCE_TRACE
#define CCE_TRACE 0
#endif
constexpr bool kTrace = CCE_TRACE != 0;


constexpr int kMaxPeers = 8;  // ranks whose memory one launch can add into

struct EngineParams {
    // extents of this launch
    int M;       // valid rows on the A side (TMEM lanes direction)
    int N;       // valid rows on the B side (TMEM columns direction)
    int K;       // reduction length
    int n_mblk;  // ceil(M / 128)
    int n_nblk;  // ceil(N / 256)
    int n_kblk;  // ceil(K / 64)
    // coordinate offsets added to the TMA coordinates of each operand
    int a_mn_off, a_k_off, b_mn_off, b_k_off;
    int a_mn_major, b_mn_major;  // 0: K contiguous in memory, 1: M/N contiguous in memory
    // MN-major operand addressed through a 3-D tensor map {64 contiguous, K rows, 64-wide groups}: one
    // TMA instruction lands every swizzle atom of a stage (else one 2-D box per 64-wide group)
    int a_tma3, b_tma3;
    uint32_t idesc;
    // Optional row count kept on the device (a caller that never read it back): when set, the
    // launch is sized on the host for the upper bound (M, or K for a product whose reduction runs
    // over the rows) and the kernel takes the real extent, min(*ptr, bound), from here.
    const long long* m_dev;
    const long long* k_dev;
    int* status;
    // optional tracing: cycles each role spent waiting, summed over CTAs (null = off)
    //   [0] producer on a free stage, [1] MMA on a filled stage, [2] MMA on a free accumulator,
    //   [3] epilogue on a finished accumulator (sum over its 4 warps / 4), [4] CTA lifetime, [5] CTAs
    unsigned long long* wait_cycles;
    // optional: CTA 0 records {clock64, globaltimer} at its start ([0], [1]) and end ([2], [3]), which
    // gives the SM clock the kernel actually ran at (null = off)
    unsigned long long* clk_words;

    // ---- MODE_LSE / MODE_PGRAD
    const float* bias;  // fp32 [>= col_off + N] or null
    int col_off;        // first local vocabulary index of this launch (chunk start)
    int has_softcap;
    float softcap;
    int band_len;       // vocabulary tiles per work item (MODE_LSE)
    float2* partial;    // [n_band][M]  (running max in log2 units, sum)
    float* tile_max;    // null or [n_mblk*4][n_nblk]: max logit (log2 units) of each 32-row x 256-col block
    // null or [N]: running maximum over all rows of each column's logit (log2 units), kept as an
    // order-preserving integer key (float_to_key) so that it can be raised with an integer atomic max
    int* col_max_key;
    // ---- block-list ("sparse") forms of the backward, used when every product is filtered:
    // only tiles that can hold a value >= eps are recomputed, each into its own slot of a pool
    // of 128x256 tiles, and the two products walk per-row / per-column lists of those slots.
    //   MODE_PGRAD, sparse != 0 : visit the slots of this pass, write G to pool slot (slot - slot_lo)
    //   MODE_GEMM,  sparse == 1 : dE[rb] += sum over the slots of row rb      (A = pool, B = classifier)
    //   MODE_GEMM,  sparse == 2 : dC[vt] = sum over the slots of column vt    (A = pool, B = embeddings)
    int sparse;
    const int* pass_info;  // device: {vt_lo, vt_hi, slot_lo, slot_hi} of this pass
    const int* slot_tile;  // [n_slots] tile id rb * n_vt + vt, sorted by vt, then rb
    const int* row_ptr;    // [n_mblk + 1] CSR over row blocks
    const int* col_ptr;    // [n_vt + 1]; column vt owns slots [col_ptr[vt], col_ptr[vt + 1])
    // K-block lists of this pass, built after phase 1 from the slot flags (klist_build_kernel):
    //   dE, row block rb : klist[4*row_ptr[rb] + i], i < kcount[rb]        = {slot_local*4 + kb, vt}
    //   dC, (vt, half h) : klist[4*col_ptr[vt] + 2*h*n + i], n = slots of vt, i < kcount[2*vt+h]
    //                                                                      = {slot_local*2 + kb, rb}
    const int2* klist;
    const int* kcount;
    int n_vt;
    uint8_t* sflag_e;  // [slot - slot_lo][4]: 64-column group of the tile has a value >= eps
    uint8_t* sflag_c;  // [slot - slot_lo][4]: (128-column half, 64-row half) has a value >= eps
    // ---- MODE_PGRAD
    const float* lse;          // [M]
    const long long* targets;  // [n_total]
    const void* valids;        // null, int32 or int64 [M]
    int valids_i64;
    long long shift;
    long long vocab_start;
    // null, or [V]: position of every (local) vocabulary index in the reordered classifier this
    // launch reads; a row's label is looked up through it
    const int* inv_order;
    const float* d_out;  // 1 element or indexed at (row + shift)
    int d_out_scalar;
    const float* d_lse;  // null or indexed at (row + shift)
    float grad_scale;
    int scale_by_inv_rows;  // multiply grad_scale by 1 / (rows of this launch): reduction "mean" with the count on the device
    float filter_eps;  // < 0: no flags are produced
    void* g_out;       // [M][ldg] 16-bit
    long long ldg;
    int g_is_bf16;
    uint8_t* flag_e;  // [n_mblk][ld_flag_e]: (128-row block, 64-column block) has a value >= eps
    int ld_flag_e;
    uint8_t* flag_c;  // [N/128][ld_flag_c]:   (128-column block, 64-row block) has a value >= eps
    int ld_flag_c;
    // ---- MODE_GEMM
    void* out;
    long long ldo;
    const int* row_map;  // null, or [M]: output row of accumulator row r (dC of a reordered classifier)
    int out_dtype;   // CCE_DT_*
    int accumulate;  // fp32 out only: 0 store, 1 read-add-store, 2 vector red.add (out pre-zeroed)
    const uint8_t* kflags;  // null or [n_mblk][ld_kflags]
    int ld_kflags;
    // Null, or a zeroed counter of this launch (block-list MODE_GEMM launches): the CTAs draw their
    // tiles from it instead of taking every gridDim.x-th one, so that a CTA that starts late or
    // meets long reductions does not hold the launch up (see TileIter).
    int* tile_counter;
    // Cross-rank sum fused into the store (dE under vocabulary parallelism): with peer_world > 0 the
    // tile of row block m is added (red.add, fp32) into the accumulator of rank m % peer_world, a
    // buffer of that rank's memory mapped into this process, at rows (m / peer_world) * 128 + r with
    // row pitch ldo.  Every rank runs the same row blocks, so each accumulator ends up with the sum
    // over ranks of the row blocks it owns.  `out` is not written.
    int peer_world;
    float* peer_out[kMaxPeers];
};

// Order-preserving map from float to int32 (and back): a < b  <=>  key(a) < key(b).
__host__ __device__ __forceinline__ int float_to_key(float f) {
#ifdef __CUDA_ARCH__
    const int b = __float_as_int(f);
#else
    int b;
    memcpy(&b, &f, 4);
#endif
    return b >= 0 ? b : (b ^ 0x7fffffff);
}
__device__ __forceinline__ float key_to_float(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }

struct EngineSmem {
    uint8_t* stages;
    uint64_t* full;    // [NSTAGE] TMA -> MMA
    uint64_t* empty;   // [NSTAGE] MMA -> TMA
    uint64_t* tfull;   // [2] MMA -> epilogue
    uint64_t* tempty;  // [2] epilogue -> MMA
    uint64_t* tdown;   // [1] tear-down
    uint32_t* tmem_base;
    int* abort_flag;
    int* acc_empty;  // [2] accumulator holds no product (all K blocks skipped)
    uint8_t* peer_stage;  // null, or PEER_STAGE_BYTES behind the barriers
    // tile queue of a launch with EngineParams::tile_counter: the producer thread draws a tile
    // number and publishes it to the MMA thread and the epilogue warps
    uint64_t* qfull;   // [TILE_QUEUE] producer -> consumers
    uint64_t* qempty;  // [TILE_QUEUE] consumers (MMA thread + 4 epilogue warps) -> producer
    int* qitem;        // [TILE_QUEUE]
};
constexpr int TILE_QUEUE = 4;
constexpr int kNoTile = 0x7fffffff;
enum { ROLE_PRODUCER = 0, ROLE_MMA = 1, ROLE_EPILOGUE = 2 };

struct PassInfo {
    int vt_lo, vt_hi, slot_lo, slot_hi;
};
// Extents that may come from the device (see EngineParams::m_dev / k_dev).
struct Dyn {
    int M, n_mblk, n_kblk;
};
__device__ __forceinline__ Dyn load_dyn(const EngineParams& p) {
    Dyn d{p.M, p.n_mblk, p.n_kblk};
    if (p.m_dev) {
        const long long m = *p.m_dev;
        d.M = int(m < 0 ? 0 : (m > p.M ? p.M : m));
        d.n_mblk = (d.M + BM - 1) / BM;
    }
    if (p.k_dev) {
        const long long k = *p.k_dev;
        const int kk = int(k < 0 ? 0 : (k > p.K ? p.K : k));
        d.n_kblk = (kk + BK - 1) / BK;
    }
    return d;
}
__device__ __forceinline__ PassInfo load_pass(const EngineParams& p) {
    PassInfo pi{0, 0, 0, 0};
    if (p.sparse) {
        pi.vt_lo = p.pass_info[0];
        pi.vt_hi = p.pass_info[1];
        pi.slot_lo = p.pass_info[2];
        pi.slot_hi = p.pass_info[3];
    }
    return pi;
}

template <int MODE>
struct TileIter {
    const EngineParams& p;
    const PassInfo& pass;
    const int n_mblk;  // row blocks of this launch (from the device when the row count lives there)
    int item, n_items, sub, sub_end;
    int mblk, nblk, band, slot;
    bool first, last;
    // tile queue (launches with p.tile_counter): set by attach()
    const EngineSmem* sm = nullptr;
    int role = 0, qslot = 0;
    uint32_t qphase = 0;
    __device__ void attach(const EngineSmem* s_, int role_) {
        sm = s_;
        role = role_;
    }
    // Next tile number of this CTA from the queue (kNoTile: none left, or a wait was abandoned).
    // The producer thread draws it from the launch's counter and publishes it; the MMA thread and
    // every epilogue thread read it and hand the queue slot back (one arrival per epilogue warp).
    __device__ int fetch() {
        int v;
        if (role == ROLE_PRODUCER) {
            if (!mbar_wait(smem_u32(&sm->qempty[qslot]), qphase ^ 1u, sm->abort_flag, p.status, ERR_WAIT_TILE_QUEUE))
                return kNoTile;
            v = atomicAdd(p.tile_counter, 1);
            if (v >= n_items) v = kNoTile;
            *reinterpret_cast<volatile int*>(&sm->qitem[qslot]) = v;
            mbar_arrive(smem_u32(&sm->qfull[qslot]));
        } else {
            if (!mbar_wait(smem_u32(&sm->qfull[qslot]), qphase, sm->abort_flag, p.status, ERR_WAIT_TILE_QUEUE))
                return kNoTile;
            v = *reinterpret_cast<volatile int*>(&sm->qitem[qslot]);
            if (role == ROLE_EPILOGUE) {
                __syncwarp();
                if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&sm->qempty[qslot]));
            } else {
                mbar_arrive(smem_u32(&sm->qempty[qslot]));
            }
        }
        if (++qslot == TILE_QUEUE) {
            qslot = 0;
            qphase ^= 1u;
        }
        return v;
    }
    __device__ TileIter(const EngineParams& p_, const PassInfo& pass_, const Dyn& dyn)
        : p(p_), pass(pass_), n_mblk(dyn.n_mblk) {
        item = int(blockIdx.x) - int(gridDim.x);
        sub = 0;
        sub_end = 0;
        slot = 0;
        if (MODE == MODE_LSE) {
            const int n_band = (p.n_nblk + p.band_len - 1) / p.band_len;
            n_items = n_band * n_mblk;
        } else if (MODE == MODE_PGRAD && p.sparse) {
            n_items = pass.slot_hi - pass.slot_lo;
        } else if (MODE == MODE_GEMM && p.sparse == 2) {
            n_items = (pass.vt_hi - pass.vt_lo) * 2 * p.n_nblk;
        } else if (MODE == MODE_GEMM && p.sparse == 1 && p.accumulate == 2 && pass.slot_lo == pass.slot_hi) {
            n_items = 0;  // an adding launch over an empty pass has nothing to add anywhere
        } else {
            n_items = n_mblk * p.n_nblk;
        }
    }
    __device__ bool next() {
        if (MODE == MODE_LSE) {
            if (sub + 1 < sub_end) {
                ++sub;
            } else {
                item += gridDim.x;
                if (item >= n_items) return false;
                band = item / n_mblk;
                mblk = item % n_mblk;
                sub = band * p.band_len;
                sub_end = min(p.n_nblk, sub + p.band_len);
            }
            nblk = sub;
            first = (sub == band * p.band_len);
            last = (sub + 1 == sub_end);
            return true;
        } else {
            if (MODE == MODE_GEMM && p.tile_counter)
                item = fetch();
            else
                item += gridDim.x;
            if (item >= n_items) return false;
            if (MODE == MODE_PGRAD) {
                if (p.sparse) {
                    const int t = p.slot_tile[pass.slot_lo + item];
                    mblk = t / p.n_vt;
                    nblk = t % p.n_vt;
                    slot = item;
                } else {
                    nblk = item / n_mblk;  // concurrent CTAs share the classifier tile
                    mblk = item % n_mblk;
                }
            } else if (p.sparse == 2) {
                mblk = pass.vt_lo * 2 + item / p.n_nblk;
                nblk = item % p.n_nblk;
            } else {
                mblk = item / p.n_nblk;
                nblk = item % p.n_nblk;
            }
            first = last = true;
            band = 0;
            return true;
        }
    }
};

// The reduction of one output tile is a list of candidate 64-element K blocks; a candidate is
// either taken (its operands are loaded and multiplied) or skipped.  Dense launches enumerate
// K blocks 0..n_kblk-1 (skipped where a flag is clear); block-list launches enumerate the
// (slot, sub-block) pairs of a row or column of the tile pool.
struct KTile {
    int n_cand;
    int e0;  // first list entry (block-list forms)
    int h;   // dC: which 128-column half of the 256-wide tile
};
struct KCoord {
    int a_mn, a_k, b_mn, b_k;
};

template <int MODE>
__device__ __forceinline__ KTile ktile_setup(const EngineParams& p, const Dyn& dyn, int mblk) {
    KTile kt{dyn.n_kblk, 0, 0};
    if (MODE == MODE_GEMM) {
        if (p.sparse == 1) {
            kt.e0 = 4 * p.row_ptr[mblk];
            kt.n_cand = p.kcount[mblk];
        } else if (p.sparse == 2) {
            const int vt = mblk >> 1;
            kt.h = mblk & 1;
            const int c0 = p.col_ptr[vt];
            kt.e0 = 4 * c0 + 2 * kt.h * (p.col_ptr[vt + 1] - c0);
            kt.n_cand = p.kcount[mblk];
        }
    }
    return kt;
}

// Where are the operands of candidate `cand` of this tile?
template <int MODE>
__device__ __forceinline__ void kcand_coords(const EngineParams& p, const KTile& kt, int mblk, int nblk, int cand,
                                             KCoord& kc) {
    if (MODE == MODE_GEMM && p.sparse == 1) {  // A = pool tile (K-major), B = classifier rows (MN-major)
        const int2 ent = p.klist[kt.e0 + cand];
        const int sl = ent.x >> 2, kb = ent.x & 3;
        kc.a_mn = sl * BM;
        kc.a_k = kb * BK;
        kc.b_mn = p.b_mn_off + nblk * BN;
        kc.b_k = ent.y * BN + kb * BK;
        return;
    }
    if (MODE == MODE_GEMM && p.sparse == 2) {  // A = pool tile (MN-major), B = embedding rows (MN-major)
        const int2 ent = p.klist[kt.e0 + cand];
        const int sl = ent.x >> 1, kb = ent.x & 1;
        kc.a_mn = kt.h * 128;
        kc.a_k = sl * BM + kb * BK;
        kc.b_mn = p.b_mn_off + nblk * BN;
        kc.b_k = ent.y * BM + kb * BK;
        return;
    }
    kc.a_mn = p.a_mn_off + mblk * BM;
    kc.a_k = p.a_k_off + cand * BK;
    kc.b_mn = p.b_mn_off + nblk * BN;
    kc.b_k = p.b_k_off + cand * BK;
}

// One thread walks the candidates a tile takes, in order, and calls fn(cand) for each; fn returns
// false to abandon the walk.  Block-list forms take every list entry; dense flagged forms read the
// skip flags of the tile's row block four at a time.  Returns the number taken, or -1 if abandoned.
// (A warp-collective walk with ballots was slower: lanes parked at a shuffle slow the one that
// issues the loads or the MMAs.)
template <int MODE, class F>
__device__ __forceinline__ int walk_taken(const EngineParams& p, const KTile& kt, int mblk, F&& fn) {
    int n = 0;
    if (MODE == MODE_GEMM && !p.sparse && p.kflags) {
        const uint8_t* f = p.kflags + (size_t)mblk * p.ld_kflags;
        int c = 0;
        if ((reinterpret_cast<uintptr_t>(f) & 3) == 0) {
            for (; c + 4 <= kt.n_cand; c += 4) {
                uint32_t w = *reinterpret_cast<const uint32_t*>(f + c);
#pragma unroll
                for (int j = 0; j < 4; ++j, w >>= 8) {
                    if (w & 0xffu) {
                        if (!fn(c + j)) return -1;
                        ++n;
                    }
                }
            }
        }
        for (; c < kt.n_cand; ++c) {
            if (f[c]) {
                if (!fn(c)) return -1;
                ++n;
            }
        }
        return n;
    }
    for (int c = 0; c < kt.n_cand; ++c) {
        if (!fn(c)) return -1;
        ++n;
    }
    return n;
}

// Operand loads of one ring stage (issued by one thread).
__device__ __forceinline__ void load_stage(const EngineParams& p, const CUtensorMap* tmA, const CUtensorMap* tmB,
                                           uint32_t sa, uint32_t sb, uint32_t bar, int a_mn, int a_k, int b_mn,
                                           int b_k) {
    if (!p.a_mn_major) {
        tma_load_2d(sa, tmA, bar, a_k, a_mn);
    } else if (p.a_tma3) {
        tma_load_3d(sa, tmA, bar, 0, a_k, a_mn >> 6);
    } else {
#pragma unroll
        for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * ATOM_BYTES, tmA, bar, a_mn + j * 64, a_k);
    }
    if (!p.b_mn_major) {
        tma_load_2d(sb, tmB, bar, b_k, b_mn);
    } else if (p.b_tma3) {
        tma_load_3d(sb, tmB, bar, 0, b_k, b_mn >> 6);
    } else {
#pragma unroll
        for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * ATOM_BYTES, tmB, bar, b_mn + j * 64, b_k);
    }
}

template <int MODE>
__device__ void producer_loop(const CUtensorMap* tmA, const CUtensorMap* tmB, const EngineParams& p,
                              const EngineSmem& s) {
    const int lane = threadIdx.x & 31;
    int stage = 0;
    uint32_t phase = 0;
    long long waited = 0;
    const PassInfo pass = load_pass(p);
    const Dyn dyn = load_dyn(p);
    TileIter<MODE> it(p, pass, dyn);
    it.attach(&s, ROLE_PRODUCER);
    const bool plain = (MODE != MODE_GEMM) || (!p.sparse && !p.kflags);  // every K block of every tile
    if (plain) {
        // One lane runs the whole loop: no ballots or shuffles on the per-K-block path.
        if (lane == 0) {
            while (it.next()) {
                const int a_mn = p.a_mn_off + it.mblk * BM, b_mn = p.b_mn_off + it.nblk * BN;
                for (int kb = 0; kb < dyn.n_kblk; ++kb) {
                    if (!mbar_wait(smem_u32(&s.empty[stage]), phase ^ 1u, s.abort_flag, p.status,
                                   ERR_WAIT_SMEM_EMPTY))
                        return;
                    const uint32_t bar = smem_u32(&s.full[stage]);
                    const uint32_t sa = smem_u32(s.stages + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
                    const int a_k = p.a_k_off + kb * BK, b_k = p.b_k_off + kb * BK;
                    mbar_expect_tx(bar, STAGE_BYTES);
                    load_stage(p, tmA, tmB, sa, sb, bar, a_mn, a_k, b_mn, b_k);
                    if (++stage == NSTAGE) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        return;
    }
    if constexpr (MODE == MODE_GEMM) {  // only the products have block-list or flagged reductions
        if (lane != 0) return;
        while (it.next()) {
            const KTile kt = ktile_setup<MODE>(p, dyn, it.mblk);
            const int taken = walk_taken<MODE>(p, kt, it.mblk, [&](int cand) -> bool {
                KCoord kc{0, 0, 0, 0};
                kcand_coords<MODE>(p, kt, it.mblk, it.nblk, cand, kc);
                const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
                if (!mbar_wait(smem_u32(&s.empty[stage]), phase ^ 1u, s.abort_flag, p.status, ERR_WAIT_SMEM_EMPTY))
                    return false;
                if (kTrace && p.wait_cycles) waited += clock64() - t0;
                const uint32_t bar = smem_u32(&s.full[stage]);
                const uint32_t sa = smem_u32(s.stages + stage * STAGE_BYTES);
                mbar_expect_tx(bar, STAGE_BYTES);
                load_stage(p, tmA, tmB, sa, sa + A_BYTES, bar, kc.a_mn, kc.a_k, kc.b_mn, kc.b_k);
                if (++stage == NSTAGE) {
                    stage = 0;
                    phase ^= 1u;
                }
                return true;
            });
            if (taken < 0) return;
        }
    }
    if (kTrace && p.wait_cycles && lane == 0) atomicAdd(p.wait_cycles + 0, (unsigned long long)waited);
}

template <int MODE>
__device__ void mma_loop(const EngineParams& p, const EngineSmem& s, uint32_t tmem_base) {
    const int lane = threadIdx.x & 31;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    // descriptor constants
    const uint32_t a_lbo = p.a_mn_major ? ATOM_BYTES : 16, b_lbo = p.b_mn_major ? ATOM_BYTES : 16;
    const uint32_t a_kstep = p.a_mn_major ? (UMMA_K / 8) * 1024 : UMMA_K * 2;  // bytes per UMMA_K
    const uint32_t b_kstep = p.b_mn_major ? (UMMA_K / 8) * 1024 : UMMA_K * 2;
    long long waited_full = 0, waited_acc = 0;
    const PassInfo pass = load_pass(p);
    const Dyn dyn = load_dyn(p);
    TileIter<MODE> it(p, pass, dyn);
    it.attach(&s, ROLE_MMA);
    const bool plain = (MODE != MODE_GEMM) || (!p.sparse && !p.kflags);  // every K block of every tile
    if (plain && dyn.n_kblk > 0) {
        if (lane == 0) {
            // descriptors of the four ring stages, built once; a K step adds to the address field
            uint64_t adesc[NSTAGE], bdesc[NSTAGE];
#pragma unroll
            for (int i = 0; i < NSTAGE; ++i) {
                const uint32_t sa = smem_u32(s.stages + i * STAGE_BYTES);
                adesc[i] = make_smem_desc(sa, a_lbo, 1024);
                bdesc[i] = make_smem_desc(sa + A_BYTES, b_lbo, 1024);
            }
            const uint64_t a_inc = a_kstep >> 4, b_inc = b_kstep >> 4;
            while (it.next()) {
                if (!mbar_wait(smem_u32(&s.tempty[acc]), acc_phase ^ 1u, s.abort_flag, p.status,
                               ERR_WAIT_TMEM_EMPTY))
                    return;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < dyn.n_kblk; ++kb) {
                    if (!mbar_wait(smem_u32(&s.full[stage]), phase, s.abort_flag, p.status, ERR_WAIT_SMEM_FULL))
                        return;
                    tc_fence_after();
                    uint64_t ad = 0, bd = 0;
#pragma unroll
                    for (int i = 0; i < NSTAGE; ++i) {  // select without dynamic register indexing
                        if (i == stage) {
                            ad = adesc[i];
                            bd = bdesc[i];
                        }
                    }
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_f16(d_tmem, ad + k * a_inc, bd + k * b_inc, p.idesc, (kb | k) ? 1u : 0u);
                    tc_commit(smem_u32(&s.empty[stage]));
                    if (++stage == NSTAGE) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                s.acc_empty[acc] = 0;
                __threadfence_block();
                tc_commit(smem_u32(&s.tfull[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        return;
    }
    if constexpr (MODE == MODE_GEMM) {  // only the products have block-list or flagged reductions
        if (lane != 0) return;
        // descriptors of the ring stages, built once; a K step adds to the address field
        uint64_t adesc[NSTAGE], bdesc[NSTAGE];
#pragma unroll
        for (int i = 0; i < NSTAGE; ++i) {
            const uint32_t sa = smem_u32(s.stages + i * STAGE_BYTES);
            adesc[i] = make_smem_desc(sa, a_lbo, 1024);
            bdesc[i] = make_smem_desc(sa + A_BYTES, b_lbo, 1024);
        }
        const uint64_t a_inc = a_kstep >> 4, b_inc = b_kstep >> 4;
        while (it.next()) {
            {
                const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
                if (!mbar_wait(smem_u32(&s.tempty[acc]), acc_phase ^ 1u, s.abort_flag, p.status, ERR_WAIT_TMEM_EMPTY))
                    return;
                if (kTrace && p.wait_cycles) waited_acc += clock64() - t0;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            int n_issued = 0;
            const KTile kt = ktile_setup<MODE>(p, dyn, it.mblk);
            const int taken = walk_taken<MODE>(p, kt, it.mblk, [&](int) -> bool {
                const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
                if (!mbar_wait(smem_u32(&s.full[stage]), phase, s.abort_flag, p.status, ERR_WAIT_SMEM_FULL))
                    return false;
                if (kTrace && p.wait_cycles) waited_full += clock64() - t0;
                tc_fence_after();
                uint64_t ad = 0, bd = 0;
#pragma unroll
                for (int i = 0; i < NSTAGE; ++i) {  // select without dynamic register indexing
                    if (i == stage) {
                        ad = adesc[i];
                        bd = bdesc[i];
                    }
                }
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_f16(d_tmem, ad + k * a_inc, bd + k * b_inc, p.idesc, (n_issued | k) ? 1u : 0u);
                tc_commit(smem_u32(&s.empty[stage]));  // frees the stage once the MMAs have read it
                ++n_issued;
                if (++stage == NSTAGE) {
                    stage = 0;
                    phase ^= 1u;
                }
                return true;
            });
            if (taken < 0) return;
            s.acc_empty[acc] = (n_issued == 0);
            __threadfence_block();
            if (n_issued)
                tc_commit(smem_u32(&s.tfull[acc]));  // arrives when the accumulator is complete
            else
                mbar_arrive(smem_u32(&s.tfull[acc]));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }
    if (kTrace && p.wait_cycles && lane == 0) {
        atomicAdd(p.wait_cycles + 1, (unsigned long long)waited_full);
        atomicAdd(p.wait_cycles + 2, (unsigned long long)waited_acc);
    }
}

__device__ __forceinline__ float apply_softcap(float x, float softcap, float inv_softcap) {
    return softcap * tanh_fast(x * inv_softcap);
}

__device__ __forceinline__ void store_g16(void* dst, const float (&v)[32], bool is_bf16) {
    uint4 o[4];
    uint32_t* w = reinterpret_cast<uint32_t*>(o);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (is_bf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {  // two full 32-byte sectors
        st_global_v8(dst, w);
        st_global_v8(reinterpret_cast<char*>(dst) + 32, w + 8);
    } else {
        uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int j = 0; j < 4; ++j) d[j] = o[j];
    }
}

// One row's 32 consecutive columns of a product tile (fp32 accumulator bits in r) to the output:
// store, read-add-store (accumulate == 1) or red.add (accumulate == 2); fp32 or 16-bit output.
// `peer` (null, or another rank's accumulator): the values are added there with red.add instead.
__device__ __forceinline__ void gemm_store_chunk(const EngineParams& p, int row, int col0, const uint32_t (&r)[32],
                                                 float* peer = nullptr) {
    float x[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]);
    const int ncol = min(32, p.N - col0);
    if (peer) {
        float* dst = peer + (size_t)row * p.ldo + col0;
        if ((ncol == 32) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) red_add_v4(dst + 4 * j, x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncol) atomicAdd(dst + j, x[j]);
        }
    } else if (p.out_dtype == 2) {
        float* dst = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldo + col0;
        const bool vec = (ncol == 32) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
        if (vec && p.accumulate == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) red_add_v4(dst + 4 * j, x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
        } else if (vec && !p.accumulate && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) st_global_v8(dst + 8 * j, r + 8 * j);
        } else if (vec) {
            float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
                if (p.accumulate) {
                    const float4 o = d4[j];
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                d4[j] = v;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncol) dst[j] = p.accumulate ? dst[j] + x[j] : x[j];
        }
    } else {
        char* dst = reinterpret_cast<char*>(p.out) + ((size_t)row * p.ldo + col0) * 2;
        const bool vec = (ncol == 32) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
        if (vec) {
            store_g16(dst, x, p.out_dtype == 1);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < ncol) {
                    if (p.out_dtype == 1)
                        reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16_rn(x[j]);
                    else
                        reinterpret_cast<__half*>(dst)[j] = __float2half_rn(x[j]);
                }
            }
        }
    }
}

// The epilogue warps' loop.  `it` walks this CTA's tiles (TileIter, or the pair form's iterator);
// tempty_bar[a] is the (shared::cluster) address of the barrier that hands accumulator a back to the
// MMA issuer, which in the two-CTA form lives in the pair's leader CTA.
template <int MODE, class Iter>
__device__ void epilogue_loop(const EngineParams& p, const EngineSmem& s, uint32_t tmem_base, Iter& it,
                              const Dyn& dyn, const uint32_t (&tempty_bar)[2]) {
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const float inv_softcap = p.has_softcap ? 1.0f / p.softcap : 0.0f;

    // MODE_LSE running state (log2 units)
    float run_m = -INFINITY, run_s = 0.0f;
    long long waited_epi = 0;

    while (it.next()) {
        const int row = it.mblk * BM + q * 32 + lane;
        const bool row_ok = row < dyn.M;

        // per-row constants (loaded before the wait so the latency overlaps the MMAs)
        float row_l2 = 0.0f, row_g = 0.0f, row_dl = 0.0f;
        int row_t = -1;
        if (MODE == MODE_PGRAD) {
            if (row_ok) {
                long long src = row;
                if (p.valids)
                    src = p.valids_i64 ? reinterpret_cast<const long long*>(p.valids)[row]
                                       : (long long)reinterpret_cast<const int*>(p.valids)[row];
                const long long ti = src + p.shift;
                const long long t = p.targets[ti] - p.vocab_start;
                row_t = (t >= 0 && t < 0x7fffffffLL) ? int(t) : -1;
                if (p.inv_order) row_t = (row_t >= 0 && row_t < p.N) ? p.inv_order[row_t] : -1;
                row_l2 = p.lse[row] * kLog2e;
                row_g = p.grad_scale * (p.d_out_scalar ? p.d_out[0] : p.d_out[ti]);
                if (p.scale_by_inv_rows) row_g /= float(dyn.M);
                row_dl = p.d_lse ? p.d_lse[ti] : 0.0f;
            }
        }
        if (MODE == MODE_LSE) {
            if (it.first) {
                run_m = -INFINITY;
                run_s = 0.0f;
            }
        }

        // every epilogue thread observes the barrier itself before touching TMEM
        const long long t0w = (kTrace && p.wait_cycles) ? clock64() : 0;
        int ok = mbar_wait(smem_u32(&s.tfull[acc]), acc_phase, s.abort_flag, p.status,
                           ERR_WAIT_TMEM_FULL);
        if (kTrace && p.wait_cycles) waited_epi += clock64() - t0w;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (MODE == MODE_GEMM && p.peer_world > 0) bulk_wait_all();
            return;
        }
        tc_fence_after();
        const bool acc_is_empty =  // every K block skipped, or a reduction of length zero
            (MODE == MODE_GEMM) ? (reinterpret_cast<volatile int*>(s.acc_empty)[acc] != 0 || dyn.n_kblk == 0) : false;
        const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);

        float tile_rowmax = -INFINITY;  // MODE_LSE: max logit (log2 units) of this row within the tile
        if (MODE == MODE_GEMM && acc_is_empty && p.accumulate) {
            // nothing to add
        } else if constexpr (MODE == MODE_GEMM) {
            if (p.peer_world > 0) {
                // The tile goes to the accumulator of the rank that owns this row block: every thread
                // stages 32 values of its row in shared memory and hands them to the copy engine as
                // one 128-byte bulk add.
                float* peer = p.peer_out[it.mblk % p.peer_world];
                const int orow = (it.mblk / p.peer_world) * BM + q * 32 + lane;
                const uint32_t stg = smem_u32(s.peer_stage) + uint32_t((q * 32 + lane) * PEER_ROW_PITCH);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = it.nblk * BN + c * 32;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint32_t r0[32];
                    tmem_ld32(taddr + c * 32, r0);
                    bulk_wait_read_all();  // the previous request has read the staging row
                    tmem_ld_wait();
                    if (row_ok) {
                        float* dst = peer + (size_t)orow * p.ldo + col0;
                        if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                st_shared_v4(stg + 16 * j, r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
                            fence_proxy_async();
                            bulk_reduce_add_f32(dst, stg, 128);
                            bulk_commit();
                        } else {
                            gemm_store_chunk(p, orow, col0, r0, peer);
                        }
                    }
                }
            } else {
                // Store-only epilogue: two 32-column loads from TMEM are in flight per wait, so half
                // of the load latency is exposed compared with one load per wait.
                const int orow = (row_ok && p.row_map) ? p.row_map[row] : row;
#pragma unroll 1
                for (int c = 0; c < BN / 32; c += 2) {
                    const int col0 = it.nblk * BN + c * 32;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint32_t r0[32], r1[32];
                    if (!acc_is_empty) {
                        tmem_ld32(taddr + c * 32, r0);
                        tmem_ld32(taddr + c * 32 + 32, r1);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
                    }
                    if (row_ok) {
                        gemm_store_chunk(p, orow, col0, r0);
                        if (col0 + 32 < p.N) gemm_store_chunk(p, orow, col0 + 32, r1);
                    }
                }
            }
        } else {
            uint32_t flag_bits = 0;  // MODE_PGRAD: activity of the current 64-column group
            // one 32-column load from TMEM per step; issuing the next chunk's load before the math of
            // this one measured +1.5 % on the recompute and -1.3 % on the forward (250 / 155 registers):
            // no gain under the power cap, so the simple form stays
            const bool from_tmem = true;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = it.nblk * BN + c * 32;  // column within this launch
                // warp-uniform; a pool slot is written in full (zeros past N) so no stale data stays in it
                if (col0 >= p.N && !(MODE == MODE_PGRAD && p.sparse)) break;
                float x[32];
                uint32_t r[32];
                if (from_tmem) {
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = from_tmem ? __uint_as_float(r[j]) : 0.0f;

                if (MODE == MODE_LSE || MODE == MODE_PGRAD) {
                    if (p.bias) {
                        const float* bp = p.bias + p.col_off + col0;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.N) x[j] += __ldg(bp + j);
                    }
                    if (p.has_softcap) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) x[j] = apply_softcap(x[j], p.softcap, inv_softcap);
                    }
                }

                if (MODE == MODE_LSE) {
                    float cmax = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        x[j] = (col0 + j < p.N) ? x[j] * kLog2e : -INFINITY;
                        cmax = fmaxf(cmax, x[j]);
                    }
                    tile_rowmax = fmaxf(tile_rowmax, cmax);
                    if (p.col_max_key) {
                        // column maxima over this warp's 32 rows: a butterfly that halves the live
                        // values at every step (31 shuffles); lane l ends up with column col0 + l
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = row_ok ? x[j] : -INFINITY;
#pragma unroll
                        for (int o = 16; o >= 1; o >>= 1) {
                            const bool up = (lane & o) != 0;
#pragma unroll
                            for (int j = 0; j < o; ++j) {
                                const float keep = up ? v[j + o] : v[j];
                                const float send = up ? v[j] : v[j + o];
                                v[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, o));
                            }
                        }
                        // one coalesced 128-byte atomic request per warp and chunk; max is order
                        // independent, so the result is the same every run
                        if (col0 + lane < p.N) atomicMax(p.col_max_key + p.col_off + col0 + lane, float_to_key(v[0]));
                    }
                    if (cmax > run_m) {
                        run_s *= ex2f(run_m - cmax);  // run_m = -inf gives 0
                        run_m = cmax;
                    }
                    if (run_m > -INFINITY) {
                        float acc_s = 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc_s += ex2f(x[j] - run_m);
                        run_s += acc_s;
                    }
                } else if (MODE == MODE_PGRAD) {
                    const float gsum = row_g + row_dl;
                    bool active = false;
                    float g[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = p.col_off + col0 + j;  // local vocabulary index
                        const bool in_range = (col0 + j < p.N);
                        float prob = in_range ? ex2f(x[j] * kLog2e - row_l2) : 0.0f;
                        const bool is_t = in_range && (col == row_t);
                        const float d0 = prob - (is_t ? 1.0f : 0.0f);
                        active |= (fabsf(d0) >= p.filter_eps);
                        float d = d0 * gsum + (is_t ? row_dl : 0.0f);
                        if (p.has_softcap) {
                            const float tt = x[j] * inv_softcap;
                            d *= (1.0f - tt * tt);
                        }
                        g[j] = row_ok ? d : 0.0f;
                    }
                    if (p.sparse) {
                        // pool slot: a dense 128x256 tile; rows past M are written as zeros
                        char* dst = reinterpret_cast<char*>(p.g_out) +
                                    (((size_t)it.slot * BM + q * 32 + lane) * BN + c * 32) * 2;
                        store_g16(dst, g, p.g_is_bf16 != 0);
                    } else if (row < p.n_mblk * BM) {
                        // rows past the count (within the buffer's blocks of 128) are stored as zeros,
                        // so that the products never meet stale values there; a CTA pair's second
                        // block may lie past the buffer altogether
                        char* dst = reinterpret_cast<char*>(p.g_out) + ((size_t)row * p.ldg + col0) * 2;
                        store_g16(dst, g, p.g_is_bf16 != 0);
                    }
                    if (p.filter_eps >= 0.0f) {
                        flag_bits |= __ballot_sync(0xffffffffu, active && row_ok);
                        // publish at the end of each 64-column group, and at the tile's last chunk
                        if ((c & 1) || (col0 + 32 >= p.N)) {
                            if (flag_bits && lane == 0) {
                                if (p.sparse) {
                                    p.sflag_e[it.slot * 4 + (c >> 1)] = 1;
                                    p.sflag_c[it.slot * 4 + (c >> 2) * 2 + (q >> 1)] = 1;
                                } else {
                                    const int cb64 = it.nblk * (BN / 64) + (c >> 1);
                                    p.flag_e[(size_t)it.mblk * p.ld_flag_e + cb64] = 1;
                                    p.flag_c[(size_t)(cb64 >> 1) * p.ld_flag_c + it.mblk * 2 + (q >> 1)] = 1;
                                }
                            }
                            flag_bits = 0;
                        }
                    }
                }
            }
        }

        // accumulator consumed: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_bar[acc]);
        if (MODE == MODE_LSE) {
            if (p.tile_max && it.mblk < dyn.n_mblk) {
                float m = row_ok ? tile_rowmax : -INFINITY;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                if (lane == 0) p.tile_max[(size_t)(it.mblk * 4 + q) * p.n_nblk + it.nblk] = m;
            }
        }
        if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
        }

        if (MODE == MODE_LSE) {
            if (it.last && row_ok) p.partial[(size_t)it.band * p.M + row] = make_float2(run_m, run_s);
        }
    }
    // bulk adds still in flight read this CTA's shared memory: they finish before the thread leaves
    if (MODE == MODE_GEMM && p.peer_world > 0) bulk_wait_all();
    if (kTrace && p.wait_cycles && lane == 0) atomicAdd(p.wait_cycles + 3, (unsigned long long)(waited_epi / 4));
}

template <int MODE>
__global__ void __launch_bounds__(ENGINE_THREADS, 1)
engine_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
              const EngineParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    EngineSmem s;
    s.stages = base;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + NSTAGE * STAGE_BYTES);
    s.full = bars;
    s.empty = bars + NSTAGE;
    s.tfull = bars + 2 * NSTAGE;
    s.tempty = bars + 2 * NSTAGE + 2;
    s.tdown = bars + 2 * NSTAGE + 4;
    s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGE + 5);
    s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
    s.acc_empty = s.abort_flag + 1;
    s.peer_stage = p.peer_world > 0 ? base + NSTAGE * STAGE_BYTES + 256 : nullptr;
    s.qfull = reinterpret_cast<uint64_t*>(base + NSTAGE * STAGE_BYTES + 128);
    s.qempty = s.qfull + TILE_QUEUE;
    s.qitem = reinterpret_cast<int*>(s.qempty + TILE_QUEUE);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long t_start = (kTrace && p.wait_cycles) ? clock64() : 0;

    {   // a CTA without a first item (a small problem, or an empty pass of the block-list backward)
        // leaves before it sets up barriers or tensor memory; the test is uniform over the CTA
        const PassInfo pass = load_pass(p);
        const TileIter<MODE> probe(p, pass, load_dyn(p));
        if (int(blockIdx.x) >= probe.n_items) return;
    }

    if (p.clk_words && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clk_words[0] = (unsigned long long)clock64();
        p.clk_words[1] = global_timer_ns();
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; ++i) {
            mbar_init(smem_u32(&s.full[i]), 1);
            mbar_init(smem_u32(&s.empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&s.tfull[i]), 1);
            mbar_init(smem_u32(&s.tempty[i]), 4);  // one arrival per epilogue warp
        }
        mbar_init(smem_u32(s.tdown), 1);
        for (int i = 0; i < TILE_QUEUE; ++i) {
            mbar_init(smem_u32(&s.qfull[i]), 1);
            mbar_init(smem_u32(&s.qempty[i]), 5);  // the MMA thread and one arrival per epilogue warp
        }
        *s.abort_flag = 0;
        s.acc_empty[0] = 0;
        s.acc_empty[1] = 0;
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(s.tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s.tmem_base);

    if (warp == 0) {
        producer_loop<MODE>(&tmA, &tmB, p, s);
    } else if (warp == 1) {
        mma_loop<MODE>(p, s, tmem_base);
    } else {
        const PassInfo pass = load_pass(p);
        const Dyn dyn = load_dyn(p);
        TileIter<MODE> it(p, pass, dyn);
        it.attach(&s, ROLE_EPILOGUE);
        const uint32_t tempty_bar[2] = {smem_u32(&s.tempty[0]), smem_u32(&s.tempty[1])};  // this CTA's own
        epilogue_loop<MODE>(p, s, tmem_base, it, dyn, tempty_bar);
    }

    // tear-down: wait (bounded) for every MMA this CTA issued, then release TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (lane == 0) {
            tc_commit(smem_u32(s.tdown));
            mbar_wait(smem_u32(s.tdown), 0, s.abort_flag, p.status, ERR_WAIT_TEARDOWN);
        }
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (p.clk_words && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clk_words[2] = (unsigned long long)clock64();
        p.clk_words[3] = global_timer_ns();
    }
    if (kTrace && p.wait_cycles && threadIdx.x == 0) {
        atomicAdd(p.wait_cycles + 4, (unsigned long long)(clock64() - t_start));
        atomicAdd(p.wait_cycles + 5, 1ull);
    }
}

}  // namespace cce
