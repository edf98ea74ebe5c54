// Forward log-sum-exp on CTA pairs (tcgen05 cta_group::2).
//
// A cluster of two CTAs computes one 256-row x 256-column logit tile per step: CTA r of the pair
// loads rows [128r, 128r+128) of the embedding block and rows [128r, 128r+128) of the classifier
// tile, the leader (rank 0) issues one M=256 MMA per K step that reads both CTAs' shared memory,
// and each CTA's TMEM receives the accumulator of its own 128 rows.  Per FLOP a CTA stages a third
// less operand data than the single-CTA pipeline (32 KB instead of 48 KB per 128x256x64 step).
// Roles per CTA as in engine.cuh: warp 0 TMA producer, warp 1 MMA issuer (leader only) and TMEM
// owner, warps 2..5 epilogue.  Same outputs as engine_kernel<MODE_LSE>.
#pragma once
#include "engine.cuh"
#include "ptx_pair.cuh"

namespace cce {

// KSUB = 64-element K sub-blocks per ring stage (1: 32 KB stages, 2: 64 KB stages), NST = ring depth
constexpr int P_SUB_BYTES = BM * BK * 2;  // one operand, 128 rows x 64 K elements (one swizzle atom column)
template <int KSUB>
struct PairCfg {
    static constexpr int NST = 6 / KSUB;
    static constexpr int A_BYTES = KSUB * P_SUB_BYTES;
    static constexpr int STAGE_BYTES = 2 * A_BYTES;
    static constexpr int SMEM = NST * STAGE_BYTES + 1024 + 256;
};
constexpr int PAIR_SMEM = PairCfg<1>::SMEM;

struct PairIter {
    const EngineParams& p;
    int item, n_items, stride, sub, sub_end;
    int rb2, nblk, band;
    bool first, last;
    __device__ PairIter(const EngineParams& p_) : p(p_) {
        stride = int(gridDim.x >> 1);
        item = int(blockIdx.x >> 1) - stride;
        sub = sub_end = 0;
        const int n_band = (p.n_nblk + p.band_len - 1) / p.band_len;
        n_items = n_band * ((p.n_mblk + 1) >> 1);
    }
    __device__ bool next() {
        if (sub + 1 < sub_end) {
            ++sub;
        } else {
            item += stride;
            if (item >= n_items) return false;
            const int n_rb2 = (p.n_mblk + 1) >> 1;
            band = item / n_rb2;
            rb2 = item % n_rb2;
            sub = band * p.band_len;
            sub_end = min(p.n_nblk, sub + p.band_len);
        }
        nblk = sub;
        first = (sub == band * p.band_len);
        last = (sub + 1 == sub_end);
        return true;
    }
};

struct PairSmem {
    uint8_t* stages;
    uint64_t* full;    // [P_NSTAGE] leader only: both CTAs' TMA bytes -> MMA
    uint64_t* empty;   // [P_NSTAGE] per CTA: MMA -> this CTA's producer
    uint64_t* tfull;   // [2] per CTA: MMA -> this CTA's epilogue
    uint64_t* tempty;  // [2] leader only: both CTAs' epilogues -> MMA
    uint64_t* tdown;
    uint32_t* tmem_base;
    int* abort_flag;
};

template <int KSUB>
__device__ void pair_producer(const CUtensorMap* tmA, const CUtensorMap* tmB, const EngineParams& p,
                              const PairSmem& s, uint32_t rank) {
    using C = PairCfg<KSUB>;
    if ((threadIdx.x & 31) != 0) return;  // one lane runs the whole loop
    int stage = 0;
    uint32_t phase = 0;
    long long waited = 0;
    PairIter it(p);
    const int n_step = (p.n_kblk + KSUB - 1) / KSUB;
    while (it.next()) {
        const int a_row = (it.rb2 * 2 + int(rank)) * BM;
        const int b_row = it.nblk * BN + int(rank) * (BN / 2);
        for (int ks = 0; ks < n_step; ++ks) {
            const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
            if (!mbar_wait(smem_u32(&s.empty[stage]), phase ^ 1u, s.abort_flag, p.status, ERR_WAIT_SMEM_EMPTY)) return;
            if (kTrace && p.wait_cycles) waited += clock64() - t0;
            const uint32_t bar_local = smem_u32(&s.full[stage]);
            const uint32_t bar_leader = map_to_cta(bar_local, 0);
            const uint32_t sa = smem_u32(s.stages + stage * C::STAGE_BYTES);
            if (rank == 0) mbar_expect_tx(bar_local, 2 * C::STAGE_BYTES);  // bytes of both CTAs
#pragma unroll
            for (int j = 0; j < KSUB; ++j) {  // columns past K are zero-filled by the tensor map
                tma_load_2d_pair(sa + j * P_SUB_BYTES, tmA, bar_leader, (ks * KSUB + j) * BK, a_row);
                tma_load_2d_pair(sa + C::A_BYTES + j * P_SUB_BYTES, tmB, bar_leader, (ks * KSUB + j) * BK, b_row);
            }
            if (++stage == C::NST) {
                stage = 0;
                phase ^= 1u;
            }
        }
    }
    if (kTrace && p.wait_cycles) atomicAdd(p.wait_cycles + 0, (unsigned long long)waited);
}

// leader CTA only; one lane runs the whole loop.  mc_commit: one multicast commit per event instead
// of one commit per CTA of the pair.
template <int KSUB>
__device__ void pair_mma(const EngineParams& p, const PairSmem& s, uint32_t tmem_base, bool mc_commit) {
    using C = PairCfg<KSUB>;
    if ((threadIdx.x & 31) != 0) return;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    long long waited_full = 0, waited_acc = 0;
    // per-stage descriptors and barrier addresses (own CTA and peer), built once
    uint64_t adesc[C::NST], bdesc[C::NST];
    uint32_t full_bar[C::NST], empty_bar[C::NST], empty_peer[C::NST];
#pragma unroll
    for (int i = 0; i < C::NST; ++i) {
        const uint32_t sa = smem_u32(s.stages + i * C::STAGE_BYTES);
        adesc[i] = make_smem_desc(sa, 16, 1024);
        bdesc[i] = make_smem_desc(sa + C::A_BYTES, 16, 1024);
        full_bar[i] = smem_u32(&s.full[i]);
        empty_bar[i] = smem_u32(&s.empty[i]);
        empty_peer[i] = map_to_cta(empty_bar[i], 1);
    }
    const uint32_t tfull_bar[2] = {smem_u32(&s.tfull[0]), smem_u32(&s.tfull[1])};
    const uint32_t tfull_peer[2] = {map_to_cta(tfull_bar[0], 1), map_to_cta(tfull_bar[1], 1)};
    PairIter it(p);
    const int n_step = (p.n_kblk + KSUB - 1) / KSUB;
    while (it.next()) {
        {
            const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
            if (!mbar_wait(smem_u32(&s.tempty[acc]), acc_phase ^ 1u, s.abort_flag, p.status, ERR_WAIT_TMEM_EMPTY))
                return;
            if (kTrace && p.wait_cycles) waited_acc += clock64() - t0;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < n_step; ++ks) {
            uint64_t ad = 0, bd = 0;
            uint32_t fb = 0, eb = 0, ep = 0;
#pragma unroll
            for (int i = 0; i < C::NST; ++i) {  // select without dynamic register indexing
                if (i == stage) {
                    ad = adesc[i];
                    bd = bdesc[i];
                    fb = full_bar[i];
                    eb = empty_bar[i];
                    ep = empty_peer[i];
                }
            }
            const long long t0 = (kTrace && p.wait_cycles) ? clock64() : 0;
            if (!mbar_wait(fb, phase, s.abort_flag, p.status, ERR_WAIT_SMEM_FULL)) return;
            if (kTrace && p.wait_cycles) waited_full += clock64() - t0;
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < KSUB; ++j) {
                const uint64_t off = uint64_t(j) * (P_SUB_BYTES >> 4);  // next 64-element K sub-block of the stage
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)  // +32 B per K step inside a swizzle row
                    tc_mma_f16_pair(d_tmem, ad + off + k * 2, bd + off + k * 2, p.idesc, (ks | j | k) ? 1u : 0u);
            }
            // the stage is free in both CTAs once these MMAs have read it
            if (mc_commit) {
                tc_commit_pair_mc(eb, 3);
            } else {
                tc_commit_pair(eb);
                tc_commit_pair(ep);
            }
            if (++stage == C::NST) {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (mc_commit) {
            tc_commit_pair_mc(acc ? tfull_bar[1] : tfull_bar[0], 3);
        } else {
            tc_commit_pair(acc ? tfull_bar[1] : tfull_bar[0]);
            tc_commit_pair(acc ? tfull_peer[1] : tfull_peer[0]);
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

__device__ void pair_epilogue(const EngineParams& p, const PairSmem& s, uint32_t tmem_base, uint32_t rank) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const float inv_softcap = p.has_softcap ? 1.0f / p.softcap : 0.0f;
    float run_m = -INFINITY, run_s = 0.0f;
    long long waited_epi = 0;
    PairIter it(p);
    while (it.next()) {
        const int mblk = it.rb2 * 2 + int(rank);
        const int row = mblk * BM + q * 32 + lane;
        const bool row_ok = row < p.M;
        if (it.first) {
            run_m = -INFINITY;
            run_s = 0.0f;
        }
        const long long t0w = (kTrace && p.wait_cycles) ? clock64() : 0;
        int ok = mbar_wait(smem_u32(&s.tfull[acc]), acc_phase, s.abort_flag, p.status, ERR_WAIT_TMEM_FULL);
        if (kTrace && p.wait_cycles) waited_epi += clock64() - t0w;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
        float tile_rowmax = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            const int col0 = it.nblk * BN + c * 32;
            if (col0 >= p.N) break;
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
            float x[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(r[j]);
            if (p.bias) {
                const float* bp = p.bias + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) x[j] += __ldg(bp + j);
            }
            if (p.has_softcap) {
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = apply_softcap(x[j], p.softcap, inv_softcap);
            }
            float cmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                x[j] = (col0 + j < p.N) ? x[j] * kLog2e : -INFINITY;
                cmax = fmaxf(cmax, x[j]);
            }
            tile_rowmax = fmaxf(tile_rowmax, cmax);
            if (cmax > run_m) {
                run_s *= ex2f(run_m - cmax);
                run_m = cmax;
            }
            if (run_m > -INFINITY) {
                float acc_s = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) acc_s += ex2f(x[j] - run_m);
                run_s += acc_s;
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s.tempty[acc]), 0));
        if (p.tile_max && mblk < p.n_mblk) {
            float m = row_ok ? tile_rowmax : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0) p.tile_max[(size_t)(mblk * 4 + q) * p.n_nblk + it.nblk] = m;
        }
        if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
        }
        if (it.last && row_ok) p.partial[(size_t)it.band * p.M + row] = make_float2(run_m, run_s);
    }
    if (kTrace && p.wait_cycles && lane == 0) atomicAdd(p.wait_cycles + 3, (unsigned long long)(waited_epi / 4));
}

template <int KSUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ENGINE_THREADS, 1)
lse_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const EngineParams p, const int mc_commit) {
    using C = PairCfg<KSUB>;
    constexpr int P_NSTAGE = C::NST;
    constexpr int P_STAGE_BYTES = C::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    PairSmem s;
    s.stages = base;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + P_NSTAGE * P_STAGE_BYTES);
    s.full = bars;
    s.empty = bars + P_NSTAGE;
    s.tfull = bars + 2 * P_NSTAGE;
    s.tempty = bars + 2 * P_NSTAGE + 2;
    s.tdown = bars + 2 * P_NSTAGE + 4;
    s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * P_NSTAGE + 5);
    s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const long long t_start = (kTrace && p.wait_cycles) ? clock64() : 0;
    if (p.clk_words && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clk_words[0] = (unsigned long long)clock64();
        p.clk_words[1] = global_timer_ns();
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < P_NSTAGE; ++i) {
            mbar_init(smem_u32(&s.full[i]), 1);
            mbar_init(smem_u32(&s.empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&s.tfull[i]), 1);
            mbar_init(smem_u32(&s.tempty[i]), 8);  // four epilogue warps in each CTA of the pair
        }
        mbar_init(smem_u32(s.tdown), 1);
        *s.abort_flag = 0;
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
        pair_producer<KSUB>(&tmA, &tmB, p, s, rank);
    } else if (warp == 1) {
        if (rank == 0) pair_mma<KSUB>(p, s, tmem_base, mc_commit != 0);
    } else {
        pair_epilogue(p, s, tmem_base, rank);
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
