// The tensor-core pipeline on CTA pairs (tcgen05 cta_group::2).
//
// A cluster of two CTAs on neighbouring SMs computes one 256 x 256 output tile per step: CTA r of
// the pair stages rows [128 r, 128 r + 128) of the A-side block and rows [128 r, 128 r + 128) of
// the B-side tile, the leader (rank 0) issues M = 256 MMAs that read both CTAs' shared memory, and
// each CTA's tensor memory receives the accumulator of its own 128 A-side rows.  Per FLOP a CTA
// stages and reads a third less operand data than the single-CTA pipeline of engine.cuh (64 KB
// instead of 96 KB per 128 x 256 x 128 step), which is what lets the tensor pipe run at its full
// rate.  A ring stage holds 128 reduction elements (two 64-element sub-blocks): with 64 per stage
// the barrier round trip per four MMAs held this form below the single-CTA one.
//
// Roles per CTA as in engine.cuh: warp 0 TMA producer (both CTAs; loads are per-CTA tiled loads
// whose bytes are credited to the leader's barrier, no cluster-wide broadcast), warp 1 MMA issuer
// (leader only) and TMEM owner, warps 2..5 epilogue (engine.cuh's epilogue_loop, unchanged).
// Serves the dense launches that take every K block: MODE_LSE, MODE_PGRAD and MODE_GEMM without
// block lists and without skip flags (a filtered product keeps the single-CTA pipeline, where a K
// block is skipped exactly when its own 128-row block has nothing above the threshold).
#pragma once
#include "engine.cuh"
#include "ptx_pair.cuh"

namespace cce {

constexpr int P_KSUB = 2;                          // 64-element K sub-blocks per ring stage
constexpr int P_NST = 3;                           // ring depth
constexpr int P_SUB_BYTES = BM * BK * 2;           // one operand, 128 rows (or columns) x 64 K elements
constexpr int P_OPER_BYTES = P_KSUB * P_SUB_BYTES;  // one operand of a stage
constexpr int P_STAGE_BYTES = 2 * P_OPER_BYTES;
constexpr int PAIR_SMEM = P_NST * P_STAGE_BYTES + 1024 + 256;

// Tiles of this pair: as TileIter, with pairs of 128-row blocks in place of single ones.
template <int MODE>
struct PairTileIter {
    const EngineParams& p;
    const int n_mblk2;  // pairs of row blocks
    const int rank;
    int item, n_items, stride, sub, sub_end;
    int mblk, mblk2, nblk, band, slot;
    bool first, last;
    __device__ PairTileIter(const EngineParams& p_, const Dyn& dyn, int rank_)
        : p(p_), n_mblk2((dyn.n_mblk + 1) >> 1), rank(rank_) {
        stride = int(gridDim.x >> 1);
        item = int(blockIdx.x >> 1) - stride;
        sub = sub_end = 0;
        slot = 0;
        if (MODE == MODE_LSE) {
            const int n_band = (p.n_nblk + p.band_len - 1) / p.band_len;
            n_items = n_band * n_mblk2;
        } else {
            n_items = n_mblk2 * p.n_nblk;
        }
    }
    __device__ bool next() {
        if (MODE == MODE_LSE) {
            if (sub + 1 < sub_end) {
                ++sub;
            } else {
                item += stride;
                if (item >= n_items) return false;
                band = item / n_mblk2;
                mblk2 = item % n_mblk2;
                sub = band * p.band_len;
                sub_end = min(p.n_nblk, sub + p.band_len);
            }
            nblk = sub;
            first = (sub == band * p.band_len);
            last = (sub + 1 == sub_end);
        } else {
            item += stride;
            if (item >= n_items) return false;
            if (MODE == MODE_PGRAD) {
                nblk = item / n_mblk2;  // concurrent pairs share the classifier tile
                mblk2 = item % n_mblk2;
            } else {
                mblk2 = item / p.n_nblk;
                nblk = item % p.n_nblk;
            }
            first = last = true;
            band = 0;
        }
        mblk = mblk2 * 2 + rank;
        return true;
    }
};

// Walks the K blocks of a tile in ascending order and hands them to `stage_fn(kbs, n)` in groups of
// up to P_KSUB (one ring stage each).  The producers of both CTAs and the MMA issuer call this with
// the same arguments and so see the same sequence of stages.  Called by one thread; stage_fn
// returns 0 to abandon the walk, and so does this.
template <class F>
__device__ __forceinline__ bool pair_walk_k(const Dyn& dyn, F&& stage_fn) {
    int kbs[P_KSUB];
    int kb = 0;
    for (; kb + P_KSUB <= dyn.n_kblk; kb += P_KSUB) {
#pragma unroll
        for (int j = 0; j < P_KSUB; ++j) kbs[j] = kb + j;
        if (!stage_fn(kbs, P_KSUB)) return false;
    }
    if (kb < dyn.n_kblk) {
        kbs[0] = kb;
        if (!stage_fn(kbs, 1)) return false;
    }
    return true;
}

template <int MODE>
__device__ void pair_producer(const CUtensorMap* tmA, const CUtensorMap* tmB, const EngineParams& p,
                              const EngineSmem& s, const Dyn& dyn, uint32_t rank) {
    if ((threadIdx.x & 31) != 0) return;  // one lane runs the whole loop
    int stage = 0;
    uint32_t phase = 0;
    long long waited = 0;
    PairTileIter<MODE> it(p, dyn, int(rank));
    while (it.next()) {
        const int a_mn = p.a_mn_off + it.mblk * BM;
        const int b_mn = p.b_mn_off + it.nblk * BN + int(rank) * (BN / 2);
        const bool ok = pair_walk_k(dyn, [&](const int* kbs, int n) -> int {
            const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
            if (!mbar_wait(smem_u32(&s.empty[stage]), phase ^ 1u, s.abort_flag, p.status, ERR_WAIT_SMEM_EMPTY)) return 0;
            if (kTrace && p.wait_cycles) waited += clock64() - t0;
            const uint32_t bar_local = smem_u32(&s.full[stage]);
            const uint32_t bar_leader = map_to_cta(bar_local, 0);
            const uint32_t sa = smem_u32(s.stages + stage * P_STAGE_BYTES);
            if (rank == 0) mbar_expect_tx(bar_local, uint32_t(n) * 4u * P_SUB_BYTES);  // both operands, both CTAs
#pragma unroll
            for (int j = 0; j < P_KSUB; ++j) {
                if (j >= n) break;
                const int a_k = p.a_k_off + kbs[j] * BK, b_k = p.b_k_off + kbs[j] * BK;
                const uint32_t da = sa + j * P_SUB_BYTES, db = sa + P_OPER_BYTES + j * P_SUB_BYTES;
                if (!p.a_mn_major)
                    tma_load_2d_pair(da, tmA, bar_leader, a_k, a_mn);
                else
                    tma_load_3d_pair(da, tmA, bar_leader, 0, a_k, a_mn >> 6);
                if (!p.b_mn_major)
                    tma_load_2d_pair(db, tmB, bar_leader, b_k, b_mn);
                else
                    tma_load_3d_pair(db, tmB, bar_leader, 0, b_k, b_mn >> 6);
            }
            if (++stage == P_NST) {
                stage = 0;
                phase ^= 1u;
            }
            return 1;
        });
        if (!ok) return;
    }
    if (kTrace && p.wait_cycles) atomicAdd(p.wait_cycles + 0, (unsigned long long)waited);
}

// leader CTA only; one lane runs the whole loop
template <int MODE>
__device__ void pair_mma(const EngineParams& p, const EngineSmem& s, const Dyn& dyn, uint32_t tmem_base) {
    if ((threadIdx.x & 31) != 0) return;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    long long waited_full = 0, waited_acc = 0;
    const uint32_t a_lbo = p.a_mn_major ? ATOM_BYTES : 16, b_lbo = p.b_mn_major ? ATOM_BYTES : 16;
    const uint64_t a_inc = (p.a_mn_major ? (UMMA_K / 8) * 1024 : UMMA_K * 2) >> 4;  // descriptor units per UMMA_K
    const uint64_t b_inc = (p.b_mn_major ? (UMMA_K / 8) * 1024 : UMMA_K * 2) >> 4;
    // per-stage descriptors and barrier addresses (own CTA and peer), built once
    uint64_t adesc[P_NST], bdesc[P_NST];
    uint32_t full_bar[P_NST], empty_bar[P_NST], empty_peer[P_NST];
#pragma unroll
    for (int i = 0; i < P_NST; ++i) {
        const uint32_t sa = smem_u32(s.stages + i * P_STAGE_BYTES);
        adesc[i] = make_smem_desc(sa, a_lbo, 1024);
        bdesc[i] = make_smem_desc(sa + P_OPER_BYTES, b_lbo, 1024);
        full_bar[i] = smem_u32(&s.full[i]);
        empty_bar[i] = smem_u32(&s.empty[i]);
        empty_peer[i] = map_to_cta(empty_bar[i], 1);
    }
    const uint32_t tfull_bar[2] = {smem_u32(&s.tfull[0]), smem_u32(&s.tfull[1])};
    const uint32_t tfull_peer[2] = {map_to_cta(tfull_bar[0], 1), map_to_cta(tfull_bar[1], 1)};
    PairTileIter<MODE> it(p, dyn, 0);
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
        const bool walked = pair_walk_k(dyn, [&](const int*, int n) -> int {
            uint64_t ad = 0, bd = 0;
            uint32_t fb = 0, eb = 0, ep = 0;
#pragma unroll
            for (int i = 0; i < P_NST; ++i) {  // select without dynamic register indexing
                if (i == stage) {
                    ad = adesc[i];
                    bd = bdesc[i];
                    fb = full_bar[i];
                    eb = empty_bar[i];
                    ep = empty_peer[i];
                }
            }
            const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
            if (!mbar_wait(fb, phase, s.abort_flag, p.status, ERR_WAIT_SMEM_FULL)) return 0;
            if (kTrace && p.wait_cycles) waited_full += clock64() - t0;
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < P_KSUB; ++j) {
                if (j >= n) break;
                const uint64_t off = uint64_t(j) * (P_SUB_BYTES >> 4);  // next K sub-block of the stage
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_f16_pair(d_tmem, ad + off + k * a_inc, bd + off + k * b_inc, p.idesc,
                                    (n_issued | j | k) ? 1u : 0u);
            }
            // the stage is free in both CTAs once these MMAs have read it
            tc_commit_pair(eb);
            tc_commit_pair(ep);
            ++n_issued;
            if (++stage == P_NST) {
                stage = 0;
                phase ^= 1u;
            }
            return 1;
        });
        if (!walked) return;
        if (n_issued) {  // arrives in both CTAs when the accumulator is complete
            tc_commit_pair(tfull_bar[acc]);
            tc_commit_pair(tfull_peer[acc]);
        } else {  // a reduction of length zero: nothing was issued, the epilogues store zeros
            mbar_arrive_cluster(tfull_bar[acc]);
            mbar_arrive_cluster(tfull_peer[acc]);
        }
        if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
        }
    }
    if (kTrace && p.wait_cycles) {
        atomicAdd(p.wait_cycles + 1, (unsigned long long)waited_full);
        atomicAdd(p.wait_cycles + 2, (unsigned long long)waited_acc);
    }
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ENGINE_THREADS, 1)
pair_engine_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const EngineParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    EngineSmem s;
    s.stages = base;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + P_NST * P_STAGE_BYTES);
    s.full = bars;             // [P_NST] leader only: both CTAs' TMA bytes -> MMA
    s.empty = bars + P_NST;    // [P_NST] per CTA: MMA -> this CTA's producer
    s.tfull = bars + 2 * P_NST;       // [2] per CTA: MMA -> this CTA's epilogue
    s.tempty = bars + 2 * P_NST + 2;  // [2] leader only: both CTAs' epilogues -> MMA
    s.tdown = bars + 2 * P_NST + 4;
    s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * P_NST + 5);
    s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
    s.acc_empty = s.abort_flag + 1;
    s.peer_stage = p.peer_world > 0 ? base + P_NST * P_STAGE_BYTES + 256 : nullptr;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const Dyn dyn = load_dyn(p);
    const long long t_start = (kTrace && p.wait_cycles) ? clock64() : 0;

    {   // a pair without a first item leaves before it sets up anything; uniform over the pair
        const PairTileIter<MODE> probe(p, dyn, 0);
        if (int(blockIdx.x >> 1) >= probe.n_items) return;
    }
    if (p.clk_words && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clk_words[0] = (unsigned long long)clock64();
        p.clk_words[1] = global_timer_ns();
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < P_NST; ++i) {
            mbar_init(smem_u32(&s.full[i]), 1);
            mbar_init(smem_u32(&s.empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&s.tfull[i]), 1);
            mbar_init(smem_u32(&s.tempty[i]), 8);  // four epilogue warps in each CTA of the pair
        }
        mbar_init(smem_u32(s.tdown), 1);
        *s.abort_flag = 0;
        s.acc_empty[0] = 0;  // an empty reduction is recognised from its length (epilogue_loop)
        s.acc_empty[1] = 0;
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(s.tmem_base), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs' barriers exist before either one signals the other
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s.tmem_base);

    if (warp == 0) {
        pair_producer<MODE>(&tmA, &tmB, p, s, dyn, rank);
    } else if (warp == 1) {
        if (rank == 0) pair_mma<MODE>(p, s, dyn, tmem_base);
    } else {
        PairTileIter<MODE> it(p, dyn, int(rank));
        const uint32_t tempty_bar[2] = {map_to_cta(smem_u32(&s.tempty[0]), 0), map_to_cta(smem_u32(&s.tempty[1]), 0)};
        epilogue_loop<MODE>(p, s, tmem_base, it, dyn, tempty_bar);
    }

    // tear-down: the leader waits (bounded) for its MMAs; neither CTA leaves, or frees TMEM, while
    // the other may still read its shared memory or signal its barriers
    tc_fence_before();
    __syncthreads();
    if (warp == 1 && rank == 0) {
        if (lane == 0) {
            tc_commit_pair(smem_u32(s.tdown));
            mbar_wait(smem_u32(s.tdown), 0, s.abort_flag, p.status, ERR_WAIT_TEARDOWN);
        }
        __syncwarp();
    }
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
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
