// Host side of the C ABI declared in include/cce_b200.h: argument checks, workspace
// planning, TMA descriptor encoding and kernel launches.  No device allocation happens here.
#include "../../include/cce_b200.h"
#include "../../include/cce_b200_testing.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "engine.cuh"
#include "engine_pair.cuh"
#include "small_kernels.cuh"

using namespace cce;

namespace {

thread_local int g_last_cuda = 0;
std::atomic<long long> g_launches{0};

#define CCE_CUDA(expr)                                   \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) {                        \
            g_last_cuda = int(e__);                      \
            return CCE_ERR_CUDA;                         \
        }                                                \
    } while (0)

#define CCE_LAUNCH_CHECK()                               \
    do {                                                 \
        g_launches.fetch_add(1);                         \
        cudaError_t e__ = cudaGetLastError();            \
        if (e__ != cudaSuccess) {                        \
            g_last_cuda = int(e__);                      \
            return CCE_ERR_CUDA;                         \
        }                                                \
    } while (0)

// Optional per-kernel timing of the tensor-core launches (off by default): one CUDA event pair
// per launch, recorded on the launch stream, summed per kernel mode when read.
struct ProfRecord {
    cudaEvent_t start, stop;
    int mode;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRecord> g_prof;
unsigned long long* g_wait_counters = nullptr;  // device memory of the caller, [3 modes][8]; null = off
unsigned long long* g_clk_words = nullptr;      // device memory of the caller, [3 modes][4]; null = off
int* g_tile_counts = nullptr;                   // device memory of the caller, 3 ints; null = off

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline long long cdiv(long long a, long long b) { return (a + b - 1) / b; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// The dense launches run on CTA pairs (engine_pair.cuh) unless CCE_B200_PAIR=0; read once.
// CCE_B200_TILE_QUEUE=0: block-list products take every gridDim.x-th tile instead of drawing from a counter
bool tile_queue_enabled() {
    static const bool on = [] {
        const char* e = getenv("CCE_B200_TILE_QUEUE");
        return !(e && e[0] == '0');
    }();
    return on;
}

bool pair_enabled() {
    static const bool on = [] {
        const char* env = getenv("CCE_B200_PAIR");
        return !(env && env[0] == '0');
    }();
    return on;
}

struct DeviceInfo {
    int sms = 0;
    int cc_major = 0;
    bool attr_set = false;
};

// Per-device facts, looked up once per device (immutable afterwards).
int device_info(DeviceInfo** out) {
    static DeviceInfo info[64];
    static std::mutex mu;
    int dev = 0;
    CCE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CCE_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo& d = info[dev];
    if (d.sms == 0) {
        CCE_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
        CCE_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    }
    if (d.cc_major != 10) return CCE_ERR_DEVICE;
    if (!d.attr_set) {
        CCE_CUDA(cudaFuncSetAttribute(engine_kernel<MODE_LSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      ENGINE_SMEM));
        CCE_CUDA(cudaFuncSetAttribute(engine_kernel<MODE_PGRAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      ENGINE_SMEM));
        CCE_CUDA(cudaFuncSetAttribute(engine_kernel<MODE_GEMM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      ENGINE_SMEM + PEER_STAGE_BYTES));
        CCE_CUDA(cudaFuncSetAttribute(pair_engine_kernel<MODE_LSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PAIR_SMEM));
        CCE_CUDA(cudaFuncSetAttribute(pair_engine_kernel<MODE_PGRAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PAIR_SMEM));
        CCE_CUDA(cudaFuncSetAttribute(pair_engine_kernel<MODE_GEMM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PAIR_SMEM + PEER_STAGE_BYTES));
        d.attr_set = true;
    }
    *out = &d;
    return CCE_OK;
}

// 2-D tensor map over a row-major 16-bit matrix: `inner` contiguous elements per row,
// `outer` rows, `pitch` elements between rows; box = box_inner x box_outer, 128-byte swizzle.
int make_tmap(CUtensorMap* m, const void* base, int dtype, long long inner, long long outer, long long pitch,
              int box_inner, int box_outer) {
    EncodeTiledFn enc = get_encode();
    if (!enc) {
        g_last_cuda = -1;
        return CCE_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch * 2) % 16) return CCE_ERR_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, dtype == CCE_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda = int(r);
        return CCE_ERR_CUDA;
    }
    return CCE_OK;
}

// 3-D tensor map over the same kind of matrix for an operand that is read MN-major (contiguous along
// M/N): dimensions {64 contiguous elements, `rows` K rows of `pitch` elements, ceil(cols/64) groups
// 128 bytes apart}, box {64, 64, box_groups}.  One load then fills `box_groups` swizzle atoms.
// The last group is read in full, so `cols` rounded up to 64 must lie inside every row's memory.
int make_tmap_mn3(CUtensorMap* m, const void* base, int dtype, long long cols, long long rows, long long pitch,
                  int box_groups) {
    EncodeTiledFn enc = get_encode();
    if (!enc) {
        g_last_cuda = -1;
        return CCE_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch * 2) % 16) return CCE_ERR_ALIGN;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)cdiv(cols, 64)};
    cuuint64_t strides[2] = {(cuuint64_t)pitch * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)BK, (cuuint32_t)box_groups};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, dtype == CCE_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda = int(r);
        return CCE_ERR_CUDA;
    }
    return CCE_OK;
}

// Map of an MN-major operand: the 3-D form when asked for (and the encoder takes it), else 2-D
// boxes of 64 x 64.  *is3 tells the kernel which one it got.
int make_tmap_mn(CUtensorMap* m, const void* base, int dtype, long long cols, long long rows, long long pitch,
                 int box_groups, bool want3, int* is3) {
    *is3 = 0;
    if (want3 && make_tmap_mn3(m, base, dtype, cols, rows, pitch, box_groups) == CCE_OK) {
        *is3 = 1;
        return CCE_OK;
    }
    return make_tmap(m, base, dtype, cols, rows, pitch, 64, BK);
}

// CCE_B200_TMA3=0 keeps every MN-major operand on 2-D boxes (for comparisons); read once.
bool tma3_enabled() {
    static const bool on = [] {
        const char* env = getenv("CCE_B200_TMA3");
        return !(env && env[0] == '0');
    }();
    return on;
}

int check_operands(const cce_b200_operands* op) {
    if (!op || !op->e || !op->c) return CCE_ERR_ARG;
    if (op->n_total < 0 || op->n_rows < 0 || op->V <= 0 || op->D <= 0) return CCE_ERR_ARG;
    if (op->n_rows > op->n_total) return CCE_ERR_ARG;
    if (!op->valids && op->n_rows != 0 && op->n_rows != op->n_total) return CCE_ERR_ARG;
    if (op->dtype != CCE_DT_F16 && op->dtype != CCE_DT_BF16 && op->dtype != CCE_DT_F32) return CCE_ERR_ARG;
    if (op->bias && (op->bias_dtype < 0 || op->bias_dtype > 2)) return CCE_ERR_ARG;
    if (op->valids && op->valids_dtype != CCE_IDX_I32 && op->valids_dtype != CCE_IDX_I64) return CCE_ERR_ARG;
    if (op->lde < op->D || op->ldc < op->D) return CCE_ERR_ARG;
    if (op->n_total >= (1LL << 31) - 256 || op->V >= (1LL << 31) - 256 || op->D >= (1LL << 30)) return CCE_ERR_ARG;
    if (op->has_softcap && !(op->softcap > 0.0f)) return CCE_ERR_ARG;
    if (op->n_rows_dev && !op->valids) return CCE_ERR_ARG;  // a count on the device comes with its row list
    return CCE_OK;
}

// Where the operands the tensor-core kernels read come from: the caller's buffers when TMA
// can address them, else packed/padded copies in the workspace.
// fp32 operands are staged as three-term bf16 splits (split_rows_kernel) and then follow the bf16 path.
inline bool is_split(const cce_b200_operands* op) { return op->dtype == CCE_DT_F32; }
inline int compute_dtype(const cce_b200_operands* op) { return is_split(op) ? CCE_DT_BF16 : op->dtype; }

struct OperandPlan {
    bool pack_e, pad_c, bias32, split, own_e;
    long long Dp;    // length (elements) of one padded block of columns, multiple of 8
    long long Drow;  // row length of the staged copies: Dp, or 3*Dp for split fp32 operands
    size_t off_e, off_c, off_bias, end;
};

// have_packed_e: the caller hands over the staged copy of e (the forward's), so none is made here
OperandPlan plan_operands(const cce_b200_operands* op, size_t start, bool have_packed_e = false) {
    OperandPlan pl;
    pl.Dp = (op->D + 7) / 8 * 8;
    const bool d_ok = (op->D % 8 == 0);
    pl.pack_e = op->valids || op->n_rows_dev || !d_ok || (op->lde % 8) || (reinterpret_cast<uintptr_t>(op->e) & 15);
    pl.pad_c = !d_ok || (op->ldc % 8) || (reinterpret_cast<uintptr_t>(op->c) & 15);
    pl.bias32 = op->bias && op->bias_dtype != CCE_DT_F32;
    pl.split = is_split(op);
    if (pl.split) pl.pack_e = pl.pad_c = true;
    pl.own_e = pl.pack_e && !have_packed_e;  // this call makes the staged copy itself
    pl.Drow = pl.split ? 3 * pl.Dp : pl.Dp;
    size_t off = align_up(start, 256);
    pl.off_e = off;
    if (pl.own_e) off = align_up(off + (size_t)op->n_rows * pl.Drow * 2, 256);
    pl.off_c = off;
    if (pl.pad_c) off = align_up(off + (size_t)op->V * pl.Drow * 2, 256);
    pl.off_bias = off;
    if (pl.bias32) off = align_up(off + (size_t)op->V * 4, 256);
    pl.end = off;
    return pl;
}

struct Staged {
    const void* e;
    long long lde;
    const void* c;
    long long ldc;
    const float* bias;
    long long Dk;   // reduction extent of E.C^T visible to TMA: D, or 3*Dp for split fp32 operands
    long long Dmn;  // extent of the column dimension when the operand is read column-major (MN-major)
    long long blk;  // distance between the column blocks of a split row (Dp), 0 otherwise
};

int stage_operands(const cce_b200_operands* op, const OperandPlan& pl, char* ws, cudaStream_t st, Staged* out,
                   const void* e_packed = nullptr) {
    const long long* ndev = reinterpret_cast<const long long*>(op->n_rows_dev);
    out->Dk = out->Dmn = op->D;
    out->blk = 0;
    if (pl.split) {
        out->Dk = out->Dmn = pl.Drow;
        out->blk = pl.Dp;
        if (op->n_rows > 0 && pl.own_e) {
            split_rows_kernel<<<(unsigned)op->n_rows, 128, 0, st>>>(
                reinterpret_cast<const float*>(op->e), op->lde, op->valids, op->valids_dtype == CCE_IDX_I64,
                reinterpret_cast<__nv_bfloat16*>(ws + pl.off_e), pl.Dp, op->D, op->n_rows, 0, ndev);
            CCE_LAUNCH_CHECK();
        }
        split_rows_kernel<<<(unsigned)op->V, 128, 0, st>>>(reinterpret_cast<const float*>(op->c), op->ldc, nullptr, 0,
                                                          reinterpret_cast<__nv_bfloat16*>(ws + pl.off_c), pl.Dp,
                                                          op->D, op->V, 1, nullptr);
        CCE_LAUNCH_CHECK();
        out->e = pl.own_e ? ws + pl.off_e : e_packed;
        out->c = ws + pl.off_c;
        out->lde = out->ldc = pl.Drow;
    } else if (pl.pack_e) {
        if (op->n_rows > 0 && pl.own_e) {
            pack_rows_kernel<<<(unsigned)op->n_rows, 128, 0, st>>>(
                reinterpret_cast<const uint16_t*>(op->e), op->lde, op->valids, op->valids_dtype == CCE_IDX_I64,
                reinterpret_cast<uint16_t*>(ws + pl.off_e), pl.Dp, op->D, op->n_rows, ndev);
            CCE_LAUNCH_CHECK();
        }
        out->e = pl.own_e ? ws + pl.off_e : e_packed;
        out->lde = pl.Dp;
    } else {
        out->e = op->e;
        out->lde = op->lde;
    }
    if (pl.split) {
        // staged above
    } else if (pl.pad_c) {
        pack_rows_kernel<<<(unsigned)op->V, 128, 0, st>>>(reinterpret_cast<const uint16_t*>(op->c), op->ldc, nullptr, 0,
                                                         reinterpret_cast<uint16_t*>(ws + pl.off_c), pl.Dp, op->D,
                                                         op->V, nullptr);
        CCE_LAUNCH_CHECK();
        out->c = ws + pl.off_c;
        out->ldc = pl.Dp;
    } else {
        out->c = op->c;
        out->ldc = op->ldc;
    }
    if (pl.bias32) {
        to_f32_kernel<<<(unsigned)cdiv(op->V, 256), 256, 0, st>>>(op->bias, op->bias_dtype,
                                                                 reinterpret_cast<float*>(ws + pl.off_bias), op->V);
        CCE_LAUNCH_CHECK();
        out->bias = reinterpret_cast<const float*>(ws + pl.off_bias);
    } else {
        out->bias = reinterpret_cast<const float*>(op->bias);
    }
    return CCE_OK;
}

int lse_band_len(long long n_rb, long long n_vt, int sms) {
    const long long want_items = (long long)sms * 8;
    const long long n_band_target = cdiv(want_items, n_rb > 0 ? n_rb : 1);
    long long len = n_vt / (n_band_target > 0 ? n_band_target : 1);
    if (len < 1) len = 1;
    if (len > 16) len = 16;
    return int(len);
}

constexpr size_t kStatusBytes = 256;
constexpr int kSmsForPlanning = 148;  // workspace sizes must not depend on the device queried later

struct LsePlan {
    OperandPlan ops;
    int band_len, n_band;
    size_t off_partial, total;
};

LsePlan plan_lse(const cce_b200_operands* op) {
    LsePlan pl;
    pl.ops = plan_operands(op, kStatusBytes);
    const long long n_rb = cdiv(op->n_rows, BM), n_vt = cdiv(op->V, BN);
    pl.band_len = lse_band_len(n_rb, n_vt, kSmsForPlanning);
    pl.n_band = int(cdiv(n_vt, pl.band_len));
    pl.off_partial = pl.ops.end;
    pl.total = align_up(pl.off_partial + (size_t)pl.n_band * op->n_rows * sizeof(float2), 256);
    return pl;
}

// pair: run on CTA pairs (dense launches only; the B-side tensor map then has boxes of 128 rows, not 256)
template <int MODE>
int launch_engine(const CUtensorMap& a, const CUtensorMap& b, const EngineParams& p, int sms, cudaStream_t st,
                  bool pair = false) {
    const long long m_units = pair ? cdiv(p.n_mblk, 2) : p.n_mblk;
    long long items;
    if (MODE == MODE_LSE)
        items = cdiv(p.n_nblk, p.band_len) * m_units;
    else
        items = m_units * p.n_nblk;
    if (items <= 0) return CCE_OK;
    const long long units = pair ? sms / 2 : sms;
    const unsigned grid = (unsigned)(items < units ? items : units) * (pair ? 2u : 1u);
    ProfRecord rec{nullptr, nullptr, MODE};
    bool prof = false;
    EngineParams pp = p;
    {
        std::lock_guard<std::mutex> lock(g_prof_mu);
        prof = g_prof_on;
        if (g_wait_counters) pp.wait_cycles = g_wait_counters + 8 * MODE;
        if (g_clk_words) pp.clk_words = g_clk_words + 4 * MODE;
    }
    if (prof) {
        CCE_CUDA(cudaEventCreate(&rec.start));
        CCE_CUDA(cudaEventCreate(&rec.stop));
        CCE_CUDA(cudaEventRecord(rec.start, st));
    }
    const size_t stage_extra = (MODE == MODE_GEMM && pp.peer_world > 0) ? PEER_STAGE_BYTES : 0;
    if (pair) {
        pp.idesc = (pp.idesc & ~(0x1fu << 24)) | ((uint32_t(2 * BM) >> 4) << 24);  // M = 256 over the pair
        pair_engine_kernel<MODE><<<grid, ENGINE_THREADS, PAIR_SMEM + stage_extra, st>>>(a, b, pp);
    } else {
        engine_kernel<MODE><<<grid, ENGINE_THREADS, ENGINE_SMEM + stage_extra, st>>>(a, b, pp);
    }
    CCE_LAUNCH_CHECK();
    if (prof) {
        CCE_CUDA(cudaEventRecord(rec.stop, st));
        std::lock_guard<std::mutex> lock(g_prof_mu);
        g_prof.push_back(rec);
    }
    return CCE_OK;
}

void base_params(EngineParams* p, long long M, long long N, long long K, int fmt, int a_mn, int b_mn, int* status) {
    memset(p, 0, sizeof(*p));
    p->M = int(M);
    p->N = int(N);
    p->K = int(K);
    p->n_mblk = int(cdiv(M, BM));
    p->n_nblk = int(cdiv(N, BN));
    p->n_kblk = int(cdiv(K, BK));
    p->a_mn_major = a_mn;
    p->b_mn_major = b_mn;
    p->idesc = make_idesc(fmt == CCE_DT_BF16 ? 1u : 0u, a_mn, b_mn, BM, BN);
    p->status = status;
    p->filter_eps = -1.0f;
    p->band_len = 1;
}

// ---- backward planning
long long gbuf_cap_bytes(bool* from_env = nullptr) {
    long long cap_bytes = 512LL << 20;
    if (from_env) *from_env = false;
    if (const char* env = getenv("CCE_B200_GBUF_MB")) {
        long long mb = atoll(env);
        if (mb >= 1) {
            cap_bytes = mb << 20;
            if (from_env) *from_env = true;
        }
    }
    return cap_bytes;
}

long long pick_chunk(long long n_rows, long long V, long long D) {
    const long long v_round = cdiv(V, BN) * BN;
    bool from_env = false;
    long long cap_bytes = gbuf_cap_bytes(&from_env);
    if (!from_env) {
        // Every vocabulary chunk costs a read-modify-write pass over the fp32 dE scratch and a round
        // of launches: a long batch gets a larger buffer (up to 2 GB) so that it needs at most 16 chunks.
        const long long for_16 = cdiv(2 * (n_rows > 0 ? n_rows : 1) * v_round, 16);
        cap_bytes = std::max(cap_bytes, std::min(for_16, 2048LL << 20));
    }
    long long cap = cap_bytes / (2 * (n_rows > 0 ? n_rows : 1)) / BN * BN;
    if (cap < BN) cap = BN;
    if (cap >= v_round) return v_round;
    // among widths within [cap/2, cap] prefer the one whose dC product fills whole waves of CTAs
    const long long n_nblk = cdiv(D, BN);
    long long best = cap;
    double best_eff = -1.0;
    for (long long w = cap; w >= BN && w * 2 >= cap; w -= BN) {
        const long long tiles = (w / BM) * n_nblk;
        const double eff = double(tiles) / double(cdiv(tiles, kSmsForPlanning) * kSmsForPlanning);
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = w;
        }
    }
    return best;
}

constexpr size_t kSlotBytes = (size_t)BM * BN * 2;  // one 128x256 16-bit tile of the pool
constexpr int kColsumRows = 512;                    // rows per block of the bias-gradient column sums

// Two shapes of the backward.
//  dense : the vocabulary is cut into chunks of Vc columns; G[B][Vc] is recomputed in full for a
//          chunk and fed to the two products.  Serves every variant.
//  sparse: when every requested product is filtered, no bias gradient is wanted and the forward's
//          per-tile maxima are at hand, only the tiles that can hold a value >= eps are
//          recomputed, into a pool of tile slots, and the products walk lists of those slots.
struct BwdPlan {
    OperandPlan ops;
    bool sparse;
    // dense
    long long Vc;  // vocabulary columns per chunk (multiple of 256)
    int n_chunk;
    int ld_flag_e, ld_flag_c;
    size_t off_flag_e, off_flag_c, flag_bytes;  // flag_e and flag_c are adjacent: one memset clears both
    size_t off_colsum;                          // [ceil(B / kColsumRows)][Vc] fp32 partial column sums (bias gradient)
    // sparse
    int n_rb, n_vt, capacity, max_pass;
    size_t off_minlse, off_act, off_col_ptr, off_row_ptr, off_slot_tile, off_slot_of, off_row_slots, off_pass,
        off_sflags, off_de_list, off_dc_list, off_de_cnt, off_dc_cnt;
    // sparse with a vocabulary order: reordered copies of the classifier (and bias), inverse order, per-tile column maxima
    bool ordered;
    long long Dkp;  // row length (elements) of the reordered classifier copy
    size_t off_cperm, off_bias_perm, off_inv_order, off_tile_colmax;
    // both
    size_t off_g, off_de32, off_tile_ctr, total;
};

bool wants_sparse(const cce_b200_backward_args* a) {
    return a->tile_max && a->has_filter && a->filter_eps > 0.0f && (!a->d_e || a->filter_e) &&
           (!a->d_c || a->filter_c) && !a->d_bias && (a->d_e || a->d_c);
}

BwdPlan plan_bwd(const cce_b200_backward_args* a) {
    const cce_b200_operands* op = &a->op;
    BwdPlan pl;
    memset(&pl, 0, sizeof(pl));
    pl.ops = plan_operands(op, kStatusBytes, a->e_packed != nullptr);
    pl.n_rb = int(cdiv(op->n_rows, BM));
    pl.n_vt = int(cdiv(op->V, BN));
    size_t off = pl.ops.end;
    pl.off_de32 = off;
    if (a->d_e) off = align_up(off + (size_t)op->n_rows * op->D * 4, 256);

    const long long total_tiles = (long long)pl.n_rb * pl.n_vt;
    long long cap = gbuf_cap_bytes() / (long long)kSlotBytes;
    if (cap > total_tiles) cap = total_tiles;
    pl.sparse = wants_sparse(a) && total_tiles > 0 && cap >= 2LL * pl.n_rb && pl.n_rb + pl.n_vt < 12000;
    if (pl.sparse) {
        pl.capacity = int(cap);
        // Every pass but the last was closed because the next column (at most n_rb tiles) did not
        // fit, so it holds at least x = cap - n_rb + 1 slots: P passes give (P - 1) * x < total, i.e.
        // P <= ceil(total / x).  A pool that holds every tile needs exactly one pass.
        pl.max_pass = cap >= total_tiles ? 1 : int(cdiv(total_tiles, cap - pl.n_rb + 1));
        pl.off_minlse = off;
        off = align_up(off + (size_t)pl.n_rb * 4 * sizeof(float), 256);
        pl.off_act = off;
        off = align_up(off + (size_t)total_tiles, 256);
        pl.off_col_ptr = off;
        off = align_up(off + (size_t)(pl.n_vt + 1) * 4, 256);
        pl.off_row_ptr = off;
        off = align_up(off + (size_t)(pl.n_rb + 1) * 4, 256);
        pl.off_slot_tile = off;
        off = align_up(off + (size_t)total_tiles * 4, 256);
        pl.off_slot_of = off;
        off = align_up(off + (size_t)total_tiles * 4, 256);
        pl.off_row_slots = off;
        off = align_up(off + (size_t)total_tiles * 4, 256);
        pl.off_pass = off;
        off = align_up(off + (size_t)pl.max_pass * 4 * sizeof(int), 256);
        pl.off_tile_ctr = off;  // [max_pass][4] tile counters of the product launches; cleared together with the flags
        off = align_up(off + (size_t)pl.max_pass * 4 * sizeof(int), 256);
        pl.off_sflags = off;  // [capacity][4] for dE, then [capacity][4] for dC
        off = align_up(off + (size_t)pl.capacity * 8, 256);
        pl.off_de_list = off;
        off = align_up(off + (size_t)total_tiles * 4 * sizeof(int2), 256);
        pl.off_dc_list = off;
        off = align_up(off + (size_t)total_tiles * 4 * sizeof(int2), 256);
        pl.off_de_cnt = off;
        off = align_up(off + (size_t)pl.n_rb * sizeof(int), 256);
        pl.off_dc_cnt = off;
        off = align_up(off + (size_t)pl.n_vt * 2 * sizeof(int), 256);
        pl.off_g = off;
        off = align_up(off + (size_t)pl.capacity * kSlotBytes, 1024);
        pl.ordered = a->vocab_order && a->col_max_key;
        if (pl.ordered) {
            const long long Dk = pl.ops.split ? pl.ops.Drow : op->D;
            pl.Dkp = (Dk + 7) / 8 * 8;
            pl.off_cperm = off;
            off = align_up(off + (size_t)op->V * pl.Dkp * 2, 256);
            pl.off_bias_perm = off;
            if (op->bias) off = align_up(off + (size_t)op->V * sizeof(float), 256);
            pl.off_inv_order = off;
            off = align_up(off + (size_t)op->V * sizeof(int), 256);
            pl.off_tile_colmax = off;
            off = align_up(off + (size_t)pl.n_vt * sizeof(float), 256);
        }
    } else {
        pl.Vc = pick_chunk(op->n_rows, op->V, op->D);
        pl.n_chunk = int(cdiv(op->V, pl.Vc));
        pl.ld_flag_e = int(pl.Vc / 64);
        pl.ld_flag_c = int(align_up((size_t)cdiv(op->n_rows, 64) + 1, 16));
        pl.off_g = off;
        off = align_up(off + (size_t)(pl.n_rb * BM) * pl.Vc * 2, 256);
        pl.off_flag_e = off;
        off = align_up(off + (size_t)pl.n_rb * pl.ld_flag_e, 256);
        pl.off_flag_c = off;
        off = align_up(off + (size_t)(pl.Vc / 128) * pl.ld_flag_c, 256);
        pl.flag_bytes = off - pl.off_flag_e;
        pl.off_colsum = off;
        if (a->d_bias) off = align_up(off + (size_t)cdiv(op->n_rows, kColsumRows) * pl.Vc * sizeof(float), 256);
    }
    pl.total = off;
    return pl;
}

}  // namespace

// Scratch of cce_b200_lse_forward_static.  In host code this name is only a handle: the device
// address is obtained per device with cudaGetSymbolAddress (static_scratch_ptr below).
static __device__ __align__(256) unsigned char g_static_scratch[CCE_B200_STATIC_SCRATCH_BYTES];

namespace {

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch_ptr(void** out) {
    static void* ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    CCE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CCE_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        CCE_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255)) return CCE_ERR_ALIGN;
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return CCE_OK;
}

}  // namespace

extern "C" {

int cce_b200_version(void) { return 1; }
int cce_b200_last_cuda_error(void) { return g_last_cuda; }
int64_t cce_b200_launch_count(void) { return (int64_t)g_launches.load(); }

const char* cce_b200_strerror(int code) {
    switch (code) {
        case CCE_OK: return "ok";
        case CCE_ERR_ARG: return "invalid argument (null pointer, bad size or unsupported dtype)";
        case CCE_ERR_ALIGN: return "pointer or stride not aligned as required";
        case CCE_ERR_WORKSPACE: return "workspace too small";
        case CCE_ERR_CUDA: return "CUDA call failed (see cce_b200_last_cuda_error)";
        case CCE_ERR_DEVICE: return "device is not sm_100";
        case CCE_ERR_KERNEL_WAIT: return "a kernel abandoned a bounded wait (status word non-zero)";
        case CCE_ERR_UNSUPPORTED: return "not available in this build of the library";
        case CCE_ERR_TOO_LARGE:
            return "problem needs more scratch than the fixed buffer of cce_b200_lse_forward_static";
        default: return "unknown error";
    }
}

int cce_b200_read_status(const void* workspace, void* stream, int32_t* word) {
    if (!workspace) return CCE_ERR_ARG;
    int32_t w = 0;
    CCE_CUDA(cudaMemcpyAsync(&w, workspace, sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    CCE_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (word) *word = w;
    return w == 0 ? CCE_OK : CCE_ERR_KERNEL_WAIT;
}

// ---- peer-shared buffers and the tail of the fused dE reduction
int cce_b200_peer_buffer_create(size_t bytes, void** ptr_out, void* handle_out) {
    if (!ptr_out || !handle_out || bytes == 0) return CCE_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == CCE_B200_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    CCE_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        CCE_CUDA(e);
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return CCE_OK;
}

int cce_b200_peer_buffer_open(const void* handle, void** ptr_out) {
    if (!handle || !ptr_out) return CCE_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    CCE_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return CCE_OK;
}

int cce_b200_peer_buffer_close(void* ptr) {
    if (!ptr) return CCE_ERR_ARG;
    CCE_CUDA(cudaIpcCloseMemHandle(ptr));
    return CCE_OK;
}

int cce_b200_peer_buffer_destroy(void* ptr) {
    if (!ptr) return CCE_ERR_ARG;
    CCE_CUDA(cudaFree(ptr));
    return CCE_OK;
}

int64_t cce_b200_de_peer_rows(int64_t n_rows, int32_t world) {
    if (n_rows < 0 || world < 1) return 0;
    return cdiv(cdiv(n_rows, BM), world) * BM;
}

int cce_b200_de_peer_collect(float* acc, int64_t acc_rows, int64_t D, void* slice_out, int32_t dtype,
                             const void* status_workspace, void* stream) {
    if (!acc || !slice_out || acc_rows < 0 || D <= 0 || acc_rows % BM != 0) return CCE_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(slice_out)) & 15) return CCE_ERR_ALIGN;
    DeviceInfo* dev = nullptr;
    int rc = device_info(&dev);
    if (rc != CCE_OK) return rc;
    const long long n = acc_rows * D;
    if (n == 0) return CCE_OK;
    const unsigned grid = (unsigned)std::min<long long>(cdiv(n / 4, 256), (long long)dev->sms * 8);
    const int* status = reinterpret_cast<const int*>(status_workspace);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CCE_DT_F32)
        peer_collect_kernel<float><<<grid, 256, 0, st>>>(acc, n, reinterpret_cast<float*>(slice_out), status);
    else if (dtype == CCE_DT_BF16)
        peer_collect_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(acc, n, reinterpret_cast<__nv_bfloat16*>(slice_out), status);
    else if (dtype == CCE_DT_F16)
        peer_collect_kernel<__half><<<grid, 256, 0, st>>>(acc, n, reinterpret_cast<__half*>(slice_out), status);
    else
        return CCE_ERR_ARG;
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

int cce_b200_de_peer_collect_push(float* acc, int64_t acc_rows, int64_t D, void* const* gather, int32_t world,
                                  int32_t rank, int32_t dtype, const void* status_workspace, void* stream) {
    if (!acc || !gather || acc_rows < 0 || D <= 0 || acc_rows % BM != 0 || world < 1 || world > kMaxPeers || rank < 0 ||
        rank >= world)
        return CCE_ERR_ARG;
    PeerPtrs ptrs{};
    for (int r = 0; r < world; ++r) {
        if (!gather[r]) return CCE_ERR_ARG;
        if (reinterpret_cast<uintptr_t>(gather[r]) & 15) return CCE_ERR_ALIGN;
        ptrs.p[r] = gather[r];
    }
    if (reinterpret_cast<uintptr_t>(acc) & 15) return CCE_ERR_ALIGN;
    DeviceInfo* dev = nullptr;
    int rc = device_info(&dev);
    if (rc != CCE_OK) return rc;
    const long long n = acc_rows * D;  // a multiple of 128
    if (n == 0) return CCE_OK;
    const int* status = reinterpret_cast<const int*>(status_workspace);
    cudaStream_t st = (cudaStream_t)stream;
    const long long per = dtype == CCE_DT_F32 ? 4 : 8;
    const unsigned grid = (unsigned)std::min<long long>(cdiv(n / per, 256), (long long)dev->sms * 8);
    if (dtype == CCE_DT_F32)
        peer_collect_push_kernel<float><<<grid, 256, 0, st>>>(acc, n, ptrs, world, rank, status);
    else if (dtype == CCE_DT_BF16)
        peer_collect_push_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(acc, n, ptrs, world, rank, status);
    else if (dtype == CCE_DT_F16)
        peer_collect_push_kernel<__half><<<grid, 256, 0, st>>>(acc, n, ptrs, world, rank, status);
    else
        return CCE_ERR_ARG;
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

int cce_b200_de_peer_scatter(const void* gathered, int32_t world, int64_t acc_rows, int64_t D, int32_t dtype,
                             const void* rows, int32_t rows_dtype, int64_t n_rows, const int64_t* n_rows_dev,
                             void* d_e, void* stream) {
    if (!gathered || !d_e || world < 1 || acc_rows < 0 || D <= 0 || n_rows < 0) return CCE_ERR_ARG;
    if (n_rows > acc_rows * world) return CCE_ERR_ARG;
    if (n_rows == 0) return CCE_OK;
    if (n_rows > 0x7fffffffLL) return CCE_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    const long long* ndev = reinterpret_cast<const long long*>(n_rows_dev);
    const int i64 = rows_dtype == CCE_IDX_I64;
    if (dtype == CCE_DT_F32)
        peer_scatter_kernel<float><<<(unsigned)n_rows, 128, 0, st>>>(reinterpret_cast<const float*>(gathered), world, acc_rows, D,
                                                                    rows, i64, reinterpret_cast<float*>(d_e), n_rows, ndev);
    else if (dtype == CCE_DT_BF16 || dtype == CCE_DT_F16)
        peer_scatter_kernel<uint16_t><<<(unsigned)n_rows, 128, 0, st>>>(reinterpret_cast<const uint16_t*>(gathered), world, acc_rows,
                                                                       D, rows, i64, reinterpret_cast<uint16_t*>(d_e), n_rows, ndev);
    else
        return CCE_ERR_ARG;
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

int cce_b200_profile_enable(int on) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_prof_on = on != 0;
    return CCE_OK;
}

int cce_b200_profile_wait_counters(void* device_counters) {
    if (device_counters && !kTrace) return CCE_ERR_UNSUPPORTED;  // this build has no tracing code
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_wait_counters = reinterpret_cast<unsigned long long*>(device_counters);
    return CCE_OK;
}

int cce_b200_profile_clock_words(void* device_words) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_clk_words = reinterpret_cast<unsigned long long*>(device_words);
    return CCE_OK;
}

int cce_b200_profile_tile_counts(void* device_counts) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_tile_counts = reinterpret_cast<int*>(device_counts);
    return CCE_OK;
}

int cce_b200_profile_read(double* ms, int64_t* launches) {
    if (!ms || !launches) return CCE_ERR_ARG;
    std::vector<ProfRecord> recs;
    {
        std::lock_guard<std::mutex> lock(g_prof_mu);
        recs.swap(g_prof);
    }
    for (int i = 0; i < 3; ++i) {
        ms[i] = 0.0;
        launches[i] = 0;
    }
    int rc = CCE_OK;
    for (ProfRecord& r : recs) {
        float t = 0.0f;
        cudaError_t e = cudaEventSynchronize(r.stop);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.start, r.stop);
        if (e != cudaSuccess) {
            g_last_cuda = int(e);
            rc = CCE_ERR_CUDA;
        } else {
            ms[r.mode] += t;
            launches[r.mode] += 1;
        }
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    return rc;
}

size_t cce_b200_lse_workspace_bytes(const cce_b200_operands* op) {
    if (check_operands(op) != CCE_OK) return 0;
    return plan_lse(op).total;
}

int cce_b200_lse_packed_e(const cce_b200_operands* op, size_t* offset, int64_t* pitch) {
    if (check_operands(op) != CCE_OK || !offset || !pitch) return CCE_ERR_ARG;
    const LsePlan pl = plan_lse(op);
    if (!pl.ops.pack_e) return 0;
    *offset = pl.ops.off_e;
    *pitch = pl.ops.Drow;
    return 1;
}

size_t cce_b200_tile_max_elems(const cce_b200_operands* op) {
    if (check_operands(op) != CCE_OK) return 0;
    return (size_t)cdiv(op->n_rows, BM) * 4 * (size_t)cdiv(op->V, BN);
}

int cce_b200_lse_forward(const cce_b200_operands* op, float* lse, float* tile_max, void* workspace,
                         size_t workspace_bytes, void* stream) {
    return cce_b200_lse_forward_ex(op, lse, tile_max, nullptr, workspace, workspace_bytes, stream);
}

int cce_b200_lse_forward_ex(const cce_b200_operands* op, float* lse, float* tile_max, int32_t* col_max_key,
                            void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_operands(op);
    if (rc != CCE_OK) return rc;
    if (!workspace || (op->n_rows > 0 && !lse)) return CCE_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return CCE_ERR_ALIGN;
    const LsePlan pl = plan_lse(op);
    if (workspace_bytes < pl.total) return CCE_ERR_WORKSPACE;
    DeviceInfo* dev = nullptr;
    rc = device_info(&dev);
    if (rc != CCE_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = reinterpret_cast<char*>(workspace);
    CCE_CUDA(cudaMemsetAsync(ws, 0, kStatusBytes, st));
    // every byte 0x80 makes each key an integer below the key of any logit (about -3.4e38 as a float)
    if (col_max_key) CCE_CUDA(cudaMemsetAsync(col_max_key, 0x80, (size_t)op->V * sizeof(int32_t), st));
    if (op->n_rows == 0) return CCE_OK;

    Staged sg;
    rc = stage_operands(op, pl.ops, ws, st, &sg);
    if (rc != CCE_OK) return rc;

    const int cdt = compute_dtype(op);
    CUtensorMap tmA, tmB;
    rc = make_tmap(&tmA, sg.e, cdt, sg.Dk, op->n_rows, sg.lde, BK, BM);
    if (rc != CCE_OK) return rc;
    rc = make_tmap(&tmB, sg.c, cdt, sg.Dk, op->V, sg.ldc, BK, BN);
    if (rc != CCE_OK) return rc;

    EngineParams p;
    base_params(&p, op->n_rows, op->V, sg.Dk, cdt, 0, 0, reinterpret_cast<int*>(ws));
    p.bias = sg.bias;
    p.has_softcap = op->has_softcap;
    p.softcap = op->softcap;
    p.band_len = pl.band_len;
    p.partial = reinterpret_cast<float2*>(ws + pl.off_partial);
    p.tile_max = tile_max;
    p.col_max_key = col_max_key;
    p.m_dev = reinterpret_cast<const long long*>(op->n_rows_dev);
    // CTA pairs need two row blocks to share a tile
    const bool pair = pair_enabled() && p.n_mblk >= 2 && dev->sms >= 2;
    if (pair) {  // each CTA of a pair stages 128 of the tile's 256 classifier rows
        rc = make_tmap(&tmB, sg.c, cdt, sg.Dk, op->V, sg.ldc, BK, BN / 2);
        if (rc != CCE_OK) return rc;
    }
    rc = launch_engine<MODE_LSE>(tmA, tmB, p, dev->sms, st, pair);
    if (rc != CCE_OK) return rc;

    lse_combine_kernel<<<(unsigned)cdiv(op->n_rows, 256), 256, 0, st>>>(p.partial, pl.n_band, op->n_rows, lse,
                                                                        reinterpret_cast<const int*>(ws), p.m_dev);
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

int cce_b200_lse_forward_static(const cce_b200_operands* op, float* lse, void* stream) {
    int rc = check_operands(op);
    if (rc != CCE_OK) return rc;
    if (plan_lse(op).total > (size_t)CCE_B200_STATIC_SCRATCH_BYTES) return CCE_ERR_TOO_LARGE;
    void* scratch = nullptr;
    rc = static_scratch_ptr(&scratch);
    if (rc != CCE_OK) return rc;
    // same launches as the workspace form; it clears the status word at the start of the scratch
    return cce_b200_lse_forward(op, lse, nullptr, scratch, (size_t)CCE_B200_STATIC_SCRATCH_BYTES, stream);
}

int cce_b200_indexed_neg_dot(const cce_b200_operands* op, const int64_t* targets, int64_t shift,
                             int64_t vocab_start, float* out, void* stream) {
    int rc = check_operands(op);
    if (rc != CCE_OK) return rc;
    if (!targets || (op->n_rows > 0 && !out) || shift < 0) return CCE_ERR_ARG;
    if (op->n_rows == 0) return CCE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const long long* ndev = reinterpret_cast<const long long*>(op->n_rows_dev);
    const unsigned blocks = (unsigned)cdiv(op->n_rows, 8);  // 8 warps per block
    if (op->dtype == CCE_DT_F32) {
        indexed_neg_dot_kernel<float><<<blocks, 256, 0, st>>>(
            reinterpret_cast<const float*>(op->e), op->lde, reinterpret_cast<const float*>(op->c), op->ldc, op->bias,
            op->bias_dtype, op->valids, op->valids_dtype == CCE_IDX_I64, reinterpret_cast<const long long*>(targets),
            shift, vocab_start, op->V, op->D, op->n_rows, op->has_softcap, op->softcap, out, ndev);
    } else if (op->dtype == CCE_DT_BF16) {
        indexed_neg_dot_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
            reinterpret_cast<const __nv_bfloat16*>(op->e), op->lde, reinterpret_cast<const __nv_bfloat16*>(op->c),
            op->ldc, op->bias, op->bias_dtype, op->valids, op->valids_dtype == CCE_IDX_I64,
            reinterpret_cast<const long long*>(targets), shift, vocab_start, op->V, op->D, op->n_rows,
            op->has_softcap, op->softcap, out, ndev);
    } else {
        indexed_neg_dot_kernel<__half><<<blocks, 256, 0, st>>>(
            reinterpret_cast<const __half*>(op->e), op->lde, reinterpret_cast<const __half*>(op->c), op->ldc,
            op->bias, op->bias_dtype, op->valids, op->valids_dtype == CCE_IDX_I64,
            reinterpret_cast<const long long*>(targets), shift, vocab_start, op->V, op->D, op->n_rows,
            op->has_softcap, op->softcap, out, ndev);
    }
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

size_t cce_b200_logit_avg_workspace_bytes(const cce_b200_operands* op) {
    if (check_operands(op) != CCE_OK) return 0;
    return align_up((size_t)(cdiv(std::max<long long>(op->n_rows, 1), kColsumRows) + 1) * op->D * sizeof(float), 256);
}

int cce_b200_logit_avg(const cce_b200_operands* op, float* out, void* workspace, size_t workspace_bytes,
                       void* stream) {
    int rc = check_operands(op);
    if (rc != CCE_OK) return rc;
    if (!out || !workspace) return CCE_ERR_ARG;
    if (workspace_bytes < cce_b200_logit_avg_workspace_bytes(op)) return CCE_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const long long B = op->n_rows, D = op->D, V = op->V;
    const int n_slices = int(cdiv(std::max<long long>(B, 1), kColsumRows));
    float* partial = reinterpret_cast<float*>(workspace);
    float* mean_e = partial + (size_t)n_slices * D;
    const dim3 grid1((unsigned)cdiv(D, 256), (unsigned)n_slices);
    const int vi64 = op->valids_dtype == CCE_IDX_I64;
    const long long* ndev = reinterpret_cast<const long long*>(op->n_rows_dev);
    const unsigned blocks3 = (unsigned)cdiv(V, 8);
#define CCE_LOGIT_AVG(T)                                                                                       \
    rows_colsum_partial_kernel<T><<<grid1, 256, 0, st>>>(reinterpret_cast<const T*>(op->e), op->lde, op->valids, \
                                                         vi64, B, D, kColsumRows, partial, ndev);              \
    CCE_LAUNCH_CHECK();                                                                                        \
    rows_colsum_finish_kernel<<<(unsigned)cdiv(D, 256), 256, 0, st>>>(partial, n_slices, D, B, mean_e, ndev);   \
    CCE_LAUNCH_CHECK();                                                                                        \
    logit_avg_kernel<T><<<blocks3, 256, 0, st>>>(mean_e, reinterpret_cast<const T*>(op->c), op->ldc, op->bias,  \
                                                 op->bias_dtype, V, D, op->has_softcap, op->softcap, out);     \
    CCE_LAUNCH_CHECK();
    if (op->dtype == CCE_DT_F32) {
        CCE_LOGIT_AVG(float)
    } else if (op->dtype == CCE_DT_BF16) {
        CCE_LOGIT_AVG(__nv_bfloat16)
    } else {
        CCE_LOGIT_AVG(__half)
    }
#undef CCE_LOGIT_AVG
    return CCE_OK;
}

int cce_b200_loss_tail(const float* stats, int32_t world, int64_t n_rows, const void* rows, int32_t rows_dtype,
                       int64_t shift, int64_t n_total, int32_t reduction, float* lse_rows, float* loss_out,
                       float* lse_scatter, const void* status_workspace, const int64_t* n_rows_dev, void* stream) {
    if (world < 1 || n_rows < 0 || n_total < n_rows || shift < 0 || reduction < 0 || reduction > 2 || !loss_out)
        return CCE_ERR_ARG;
    if (n_rows > 0 && !stats) return CCE_ERR_ARG;
    if (rows && rows_dtype != CCE_IDX_I32 && rows_dtype != CCE_IDX_I64) return CCE_ERR_ARG;
    if (!rows && n_rows != n_total && n_rows != 0) return CCE_ERR_ARG;
    if (n_rows_dev && !rows) return CCE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const bool scattered = rows != nullptr || n_rows != n_total;  // some positions receive no row: clear them first
    if (scattered && n_total > 0) {
        if (reduction == 2) CCE_CUDA(cudaMemsetAsync(loss_out, 0, (size_t)n_total * sizeof(float), st));
        if (lse_scatter) CCE_CUDA(cudaMemsetAsync(lse_scatter, 0, (size_t)n_total * sizeof(float), st));
    }
    if (n_rows == 0 && reduction == 2) return CCE_OK;  // (an upper bound of 0 leaves nothing to scatter either)
    loss_tail_kernel<<<TAIL_CTAS, TAIL_THREADS, 0, st>>>(stats, world, n_rows, rows, rows_dtype == CCE_IDX_I64, shift, reduction,
                                                 lse_rows, loss_out, lse_scatter,
                                                 reinterpret_cast<const int*>(status_workspace),
                                                 reinterpret_cast<const long long*>(n_rows_dev));
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

size_t cce_b200_valid_rows_workspace_bytes(int64_t n_total) {
    if (n_total < 0) return 0;
    return align_up((size_t)cdiv(std::max<long long>(n_total, 1), VR_BLOCK) * sizeof(int), 256);
}

int cce_b200_valid_rows(const int64_t* targets, int64_t n_total, int64_t seq_len, int64_t shift,
                        int64_t ignore_index, void* rows_out, int rows_dtype, int64_t* count_out, void* workspace,
                        size_t workspace_bytes, void* stream) {
    if (!count_out || n_total < 0 || shift < 0 || seq_len <= 0 || n_total % seq_len != 0) return CCE_ERR_ARG;
    if (rows_dtype != CCE_IDX_I32 && rows_dtype != CCE_IDX_I64) return CCE_ERR_ARG;
    if (rows_dtype == CCE_IDX_I32 && n_total > 0x7fffffffLL) return CCE_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_total == 0 || shift >= seq_len) {
        set_count_kernel<<<1, 1, 0, st>>>(reinterpret_cast<long long*>(count_out), 0);  // count_out may be host-mapped
        CCE_LAUNCH_CHECK();
        return CCE_OK;
    }
    if (!targets || !rows_out || !workspace) return CCE_ERR_ARG;
    if (workspace_bytes < cce_b200_valid_rows_workspace_bytes(n_total)) return CCE_ERR_WORKSPACE;
    const long long blocks = cdiv(n_total, VR_BLOCK);
    if (blocks > 0x7fffffffLL) return CCE_ERR_TOO_LARGE;
    int* block_counts = reinterpret_cast<int*>(workspace);
    const long long* t = reinterpret_cast<const long long*>(targets);
    valid_rows_count_kernel<<<(unsigned)blocks, VR_THREADS, 0, st>>>(t, n_total, seq_len, shift, ignore_index,
                                                                      block_counts);
    CCE_LAUNCH_CHECK();
    valid_rows_write_kernel<<<(unsigned)blocks, VR_THREADS, 0, st>>>(
        t, n_total, seq_len, shift, ignore_index, block_counts, rows_out, rows_dtype == CCE_IDX_I64,
        reinterpret_cast<long long*>(count_out));
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

size_t cce_b200_backward_workspace_bytes(const cce_b200_backward_args* a) {
    if (!a || check_operands(&a->op) != CCE_OK) return 0;
    return plan_bwd(a).total;
}

int cce_b200_backward(const cce_b200_backward_args* a, void* workspace, size_t workspace_bytes, void* stream) {
    if (!a) return CCE_ERR_ARG;
    const cce_b200_operands* op = &a->op;
    int rc = check_operands(op);
    if (rc != CCE_OK) return rc;
    if (!workspace || !a->targets || !a->d_out || a->shift < 0) return CCE_ERR_ARG;
    if (op->n_rows > 0 && !a->lse) return CCE_ERR_ARG;
    if (a->d_out_numel != 1 && a->d_out_numel != op->n_total) return CCE_ERR_ARG;
    if (a->d_bias && !op->bias) return CCE_ERR_ARG;
    if (a->has_filter && !(a->filter_eps >= 0.0f)) return CCE_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return CCE_ERR_ALIGN;
    const int peer_world = a->de_peer_world > 1 ? a->de_peer_world : 0;  // dE added into the ranks' accumulators
    if (peer_world) {
        if (peer_world > kMaxPeers || !a->d_e) return CCE_ERR_ARG;
        for (int r = 0; r < peer_world; ++r)
            if (!a->de_peer_acc[r] || (reinterpret_cast<uintptr_t>(a->de_peer_acc[r]) & 15)) return CCE_ERR_ARG;
    }
    const BwdPlan pl = plan_bwd(a);
    if (workspace_bytes < pl.total) return CCE_ERR_WORKSPACE;
    DeviceInfo* dev = nullptr;
    rc = device_info(&dev);
    if (rc != CCE_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = reinterpret_cast<char*>(workspace);
    const long long D = op->D, V = op->V, B = op->n_rows;  // B: the row count, or its upper bound when the count is on the device
    const long long* ndev = reinterpret_cast<const long long*>(op->n_rows_dev);
    const int cdt = compute_dtype(op);      // type the tensor cores see (fp32 operands are split into bf16)
    const bool split = is_split(op);
    const size_t esz = split ? 4 : 2;       // element size of the caller's e, c, d_c (and d_e unless d_e_f32)

    CCE_CUDA(cudaMemsetAsync(ws, 0, kStatusBytes, st));
    const size_t de_esz = (a->d_e_f32 || split) ? 4 : esz;
    if (a->d_e && (op->valids || B == 0)) CCE_CUDA(cudaMemsetAsync(a->d_e, 0, (size_t)op->n_total * D * de_esz, st));
    if (B == 0) {
        if (a->d_bias) CCE_CUDA(cudaMemsetAsync(a->d_bias, 0, (size_t)V * 4, st));
        if (a->d_c) CCE_CUDA(cudaMemsetAsync(a->d_c, 0, (size_t)V * D * esz, st));
        return CCE_OK;
    }

    if (a->e_packed && pl.ops.pack_e &&
        (a->e_packed_ld != pl.ops.Drow || (reinterpret_cast<uintptr_t>(a->e_packed) & 15)))
        return CCE_ERR_ARG;  // not the staged copy cce_b200_lse_packed_e describes
    Staged sg;
    rc = stage_operands(op, pl.ops, ws, st, &sg, a->e_packed);
    if (rc != CCE_OK) return rc;

    // A vocabulary order (block-list form only): the products and the recomputation read a copy of the
    // classifier (and bias) whose rows are in that order, labels are looked up through the inverse
    // order, and dC rows are stored back at their own positions.
    int* inv_order = nullptr;
    float* tile_colmax = nullptr;
    if (pl.sparse && pl.ordered) {
        inv_order = reinterpret_cast<int*>(ws + pl.off_inv_order);
        tile_colmax = reinterpret_cast<float*>(ws + pl.off_tile_colmax);
        order_prepare_kernel<<<(unsigned)pl.n_vt, 256, 0, st>>>(a->vocab_order, V, a->col_max_key, inv_order, tile_colmax);
        CCE_LAUNCH_CHECK();
        pack_rows_kernel<<<(unsigned)V, 128, 0, st>>>(reinterpret_cast<const uint16_t*>(sg.c), sg.ldc, a->vocab_order, 0,
                                                     reinterpret_cast<uint16_t*>(ws + pl.off_cperm), pl.Dkp, sg.Dk, V, nullptr);
        CCE_LAUNCH_CHECK();
        sg.c = ws + pl.off_cperm;
        sg.ldc = pl.Dkp;
        if (sg.bias) {
            float* bias_perm = reinterpret_cast<float*>(ws + pl.off_bias_perm);
            gather_f32_kernel<<<(unsigned)cdiv(V, 256), 256, 0, st>>>(sg.bias, CCE_DT_F32, a->vocab_order, bias_perm, V);
            CCE_LAUNCH_CHECK();
            sg.bias = bias_perm;
        }
    }

    const bool use_flags = a->has_filter && ((a->filter_e && a->d_e) || (a->filter_c && a->d_c));
    int* status = reinterpret_cast<int*>(ws);
    char* g_buf = ws + pl.off_g;
    float* de32 = reinterpret_cast<float*>(ws + pl.off_de32);

    // operand maps that do not change from chunk to chunk
    CUtensorMap tmE_k, tmC_k, tmE_mn, tmC_mn;
    rc = make_tmap(&tmE_k, sg.e, cdt, sg.Dk, B, sg.lde, BK, BM);
    if (rc != CCE_OK) return rc;
    rc = make_tmap(&tmC_k, sg.c, cdt, sg.Dk, V, sg.ldc, BK, BN);
    if (rc != CCE_OK) return rc;
    // MN-major views (for G^T E and G C): one 3-D load per stage when the rows are whole 64-element groups
    const bool mn3 = tma3_enabled() && sg.Dmn % 64 == 0 && (!split || sg.blk % 64 == 0);
    int e_is3 = 0, c_is3 = 0;
    rc = make_tmap_mn(&tmE_mn, sg.e, cdt, sg.Dmn, B, sg.lde, BN / 64, mn3, &e_is3);
    if (rc != CCE_OK) return rc;
    rc = make_tmap_mn(&tmC_mn, sg.c, cdt, sg.Dmn, V, sg.ldc, BN / 64, mn3, &c_is3);
    if (rc != CCE_OK) return rc;

    // Dense launches that take every K block run on CTA pairs: each CTA stages 128 of the B side's 256 rows
    const bool can_pair = pair_enabled() && !pl.sparse && dev->sms >= 2;
    CUtensorMap tmC_k_h, tmE_mn_h, tmC_mn_h;
    if (can_pair) {
        int is3 = 0;
        rc = make_tmap(&tmC_k_h, sg.c, cdt, sg.Dk, V, sg.ldc, BK, BN / 2);
        if (rc != CCE_OK) return rc;
        if (e_is3) rc = make_tmap_mn(&tmE_mn_h, sg.e, cdt, sg.Dmn, B, sg.lde, BN / 128, true, &is3);
        if (rc != CCE_OK) return rc;
        if (c_is3) rc = make_tmap_mn(&tmC_mn_h, sg.c, cdt, sg.Dmn, V, sg.ldc, BN / 128, true, &is3);
        if (rc != CCE_OK) return rc;
    }
    // a product runs on pairs when nothing is skipped, both MN-major operands have 3-D maps, and two row blocks exist
    auto pair_ok = [&](const EngineParams& p, int b_is3) {
        return can_pair && !p.kflags && !p.sparse && p.n_mblk >= 2 && b_is3 && (!p.a_mn_major || p.a_tma3);
    };

    // The two products.  With split fp32 operands the staged rows hold three column blocks
    // ([hi|hi|lo] for e, [hi|lo|hi] for c): dC = G^T e_hi + G^T e_lo and dE = G c_hi + G c_lo, i.e. the
    // same launch run twice on different column blocks of the B operand, the second adding in fp32.
    // SMs the dC product may use: all of them, except after dE has been handed to the caller's
    // exchange (finish_de), which needs SMs of its own to run beside the product
    int sms_dc = dev->sms;
    auto run_dc = [&](EngineParams p, const CUtensorMap& tmA) -> int {
        p.b_tma3 = e_is3;
        const bool pair = pair_ok(p, e_is3);
        const CUtensorMap& tmB = pair ? tmE_mn_h : tmE_mn;
        int r = launch_engine<MODE_GEMM>(tmA, tmB, p, sms_dc, st, pair);
        if (r != CCE_OK || !split) return r;
        p.b_mn_off = int(2 * sg.blk);
        p.accumulate = 2;
        if (p.tile_counter) ++p.tile_counter;
        return launch_engine<MODE_GEMM>(tmA, tmB, p, sms_dc, st, pair);
    };
    auto run_de = [&](EngineParams p, const CUtensorMap& tmA) -> int {
        p.b_tma3 = c_is3;
        const bool pair = pair_ok(p, c_is3);
        const CUtensorMap& tmB = pair ? tmC_mn_h : tmC_mn;
        int r = launch_engine<MODE_GEMM>(tmA, tmB, p, dev->sms, st, pair);
        if (r != CCE_OK || !split) return r;
        p.b_mn_off = int(sg.blk);
        p.accumulate = 2;
        if (p.tile_counter) ++p.tile_counter;
        return launch_engine<MODE_GEMM>(tmA, tmB, p, dev->sms, st, pair);
    };

    // phase-1 parameters shared by both shapes
    EngineParams pg;
    base_params(&pg, B, V, sg.Dk, cdt, 0, 0, status);
    pg.bias = sg.bias;
    pg.has_softcap = op->has_softcap;
    pg.softcap = op->softcap;
    pg.lse = a->lse;
    pg.targets = reinterpret_cast<const long long*>(a->targets);
    pg.valids = op->valids;
    pg.valids_i64 = op->valids_dtype == CCE_IDX_I64;
    pg.shift = a->shift;
    pg.vocab_start = a->vocab_start;
    pg.d_out = a->d_out;
    pg.d_out_scalar = a->d_out_numel == 1;
    pg.d_lse = a->d_lse;
    pg.grad_scale = a->grad_scale;
    pg.scale_by_inv_rows = a->grad_scale_by_inv_rows;
    pg.m_dev = ndev;
    pg.filter_eps = use_flags ? a->filter_eps : -1.0f;
    pg.g_out = g_buf;
    pg.g_is_bf16 = cdt == CCE_DT_BF16;
    pg.inv_order = inv_order;

    // The last step of dE: fp32 scratch -> the caller's rows.  Run once, either at the end or, when the
    // caller asked to be told (de_ready_event), right after the last dE product and before the last dC
    // product, so that a cross-rank reduction of dE can overlap that product.
    const bool early_de = a->d_e && (a->de_ready_event != nullptr || peer_world);
    bool de_finished = false;
    auto set_peers = [&](EngineParams& p) {  // the dE product adds into the owners' accumulators
        if (!peer_world) return;
        p.peer_world = peer_world;
        for (int r = 0; r < peer_world; ++r) p.peer_out[r] = a->de_peer_acc[r];
        p.accumulate = 2;
    };
    auto finish_de = [&]() -> int {
        if (de_finished || !a->d_e) return CCE_OK;
        de_finished = true;
        if (a->de_ready_event && a->exchange_sms > 0)
            sms_dc = std::max(dev->sms / 2, dev->sms - a->exchange_sms) & ~1;  // even: CTA pairs
        if (peer_world) {  // the sums sit in the ranks' accumulators: the caller collects them
            if (a->de_ready_event) CCE_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(a->de_ready_event), st));
            return CCE_OK;
        }
        if (a->d_e_f32 || split)
            scatter_cast_kernel<float><<<(unsigned)B, 128, 0, st>>>(
                de32, D, op->valids, op->valids_dtype == CCE_IDX_I64, reinterpret_cast<float*>(a->d_e), D, D, B, status, ndev);
        else if (cdt == CCE_DT_BF16)
            scatter_cast_kernel<__nv_bfloat16><<<(unsigned)B, 128, 0, st>>>(
                de32, D, op->valids, op->valids_dtype == CCE_IDX_I64, reinterpret_cast<__nv_bfloat16*>(a->d_e), D, D, B,
                status, ndev);
        else
            scatter_cast_kernel<__half><<<(unsigned)B, 128, 0, st>>>(
                de32, D, op->valids, op->valids_dtype == CCE_IDX_I64, reinterpret_cast<__half*>(a->d_e), D, D, B, status, ndev);
        CCE_LAUNCH_CHECK();
        if (a->de_ready_event) CCE_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(a->de_ready_event), st));
        return CCE_OK;
    };

    if (pl.sparse) {
        // ---- index of the tiles worth recomputing
        const int n_groups = pl.n_rb * 4;
        float* minlse = reinterpret_cast<float*>(ws + pl.off_minlse);
        uint8_t* act = reinterpret_cast<uint8_t*>(ws + pl.off_act);
        int* col_ptr = reinterpret_cast<int*>(ws + pl.off_col_ptr);
        int* row_ptr = reinterpret_cast<int*>(ws + pl.off_row_ptr);
        int* slot_tile = reinterpret_cast<int*>(ws + pl.off_slot_tile);
        int* slot_of = reinterpret_cast<int*>(ws + pl.off_slot_of);
        int* row_slots = reinterpret_cast<int*>(ws + pl.off_row_slots);
        int* pass_info = reinterpret_cast<int*>(ws + pl.off_pass);
        uint8_t* sflag_e = reinterpret_cast<uint8_t*>(ws + pl.off_sflags);
        uint8_t* sflag_c = sflag_e + (size_t)pl.capacity * 4;
        int2* de_list = reinterpret_cast<int2*>(ws + pl.off_de_list);
        int2* dc_list = reinterpret_cast<int2*>(ws + pl.off_dc_list);
        int* de_cnt = reinterpret_cast<int*>(ws + pl.off_de_cnt);
        int* dc_cnt = reinterpret_cast<int*>(ws + pl.off_dc_cnt);
        CCE_CUDA(cudaMemsetAsync(act, 0, (size_t)pl.n_rb * pl.n_vt, st));
        rowgroup_min_lse_kernel<<<(unsigned)cdiv(n_groups, 8), 256, 0, st>>>(a->lse, B, minlse, n_groups, ndev);
        CCE_LAUNCH_CHECK();
        if (inv_order) {
            const long long n_thr = std::max<long long>(B, (long long)n_groups * pl.n_vt * 32);
            tile_mark_ordered_kernel<<<(unsigned)cdiv(n_thr, 256), 256, 0, st>>>(
                a->tile_max, minlse, tile_colmax, a->vocab_order, inv_order, n_groups, pl.n_vt, log2f(a->filter_eps),
                reinterpret_cast<const long long*>(a->targets), op->valids, op->valids_dtype == CCE_IDX_I64, a->shift,
                a->vocab_start, V, B, act, ndev);
        } else {
            const long long n_thr = std::max<long long>(B, (long long)n_groups * pl.n_vt);
            tile_mark_kernel<<<(unsigned)cdiv(n_thr, 256), 256, 0, st>>>(
                a->tile_max, minlse, n_groups, pl.n_vt, log2f(a->filter_eps),
                reinterpret_cast<const long long*>(a->targets), op->valids, op->valids_dtype == CCE_IDX_I64, a->shift,
                a->vocab_start, V, B, act, ndev);
        }
        CCE_LAUNCH_CHECK();
        const size_t sm_bytes = (size_t)(pl.n_rb + pl.n_vt + 2) * sizeof(int);
        int* tile_counts = nullptr;
        {
            std::lock_guard<std::mutex> lock(g_prof_mu);
            tile_counts = g_tile_counts;
        }
        tile_index_kernel<<<1, 1024, sm_bytes, st>>>(act, pl.n_rb, pl.n_vt, pl.capacity, pl.max_pass, col_ptr, slot_tile,
                                                    slot_of, row_ptr, row_slots, pass_info, tile_counts, B, ndev);
        CCE_LAUNCH_CHECK();

        CUtensorMap tmP_k, tmP_mn;  // the pool seen as a [capacity*128][256] matrix
        rc = make_tmap(&tmP_k, g_buf, cdt, BN, (long long)pl.capacity * BM, BN, BK, BM);
        if (rc != CCE_OK) return rc;
        int p_is3 = 0;
        rc = make_tmap_mn(&tmP_mn, g_buf, cdt, BN, (long long)pl.capacity * BM, BN, BM / 64, tma3_enabled(), &p_is3);
        if (rc != CCE_OK) return rc;

        // slot flags (later passes: cleared by their reader) and, in front of them, the tile counters
        int* tile_ctr = tile_queue_enabled() ? reinterpret_cast<int*>(ws + pl.off_tile_ctr) : nullptr;
        CCE_CUDA(cudaMemsetAsync(ws + pl.off_tile_ctr, 0, (pl.off_sflags - pl.off_tile_ctr) + (size_t)pl.capacity * 8, st));
        for (int ps = 0; ps < pl.max_pass; ++ps) {
            const int* pinfo = pass_info + 4 * ps;
            {
                EngineParams p = pg;
                p.sparse = 1;
                p.pass_info = pinfo;
                p.slot_tile = slot_tile;
                p.n_vt = pl.n_vt;
                p.sflag_e = sflag_e;
                p.sflag_c = sflag_c;
                rc = launch_engine<MODE_PGRAD>(tmE_k, tmC_k, p, dev->sms, st);
                if (rc != CCE_OK) return rc;
            }
            klist_build_kernel<<<(unsigned)cdiv(pl.n_rb + 2 * pl.n_vt, 8), 256, 0, st>>>(
                pinfo, row_ptr, row_slots, col_ptr, slot_tile, pl.n_rb, pl.n_vt, sflag_e, sflag_c, de_list, de_cnt,
                dc_list, dc_cnt);
            CCE_LAUNCH_CHECK();
            auto pass_dc = [&]() -> int {  // dC[vt] = sum over the slots of column vt of G^T E
                if (!a->d_c) return CCE_OK;
                EngineParams p;
                base_params(&p, V, D, B, cdt, 1, 1, status);
                p.out = a->d_c;
                p.ldo = D;
                p.out_dtype = split ? CCE_DT_F32 : op->dtype;
                p.accumulate = 0;
                p.sparse = 2;
                p.pass_info = pinfo;
                p.slot_tile = slot_tile;
                p.col_ptr = col_ptr;
                p.n_vt = pl.n_vt;
                p.klist = dc_list;
                p.kcount = dc_cnt;
                p.a_tma3 = p_is3;
                p.row_map = inv_order ? a->vocab_order : nullptr;
                if (tile_ctr) p.tile_counter = tile_ctr + 4 * ps;
                return run_dc(p, tmP_mn);
            };
            auto pass_de = [&]() -> int {  // dE[rb] += sum over the slots of row rb (in this pass) of G C
                if (!a->d_e) return CCE_OK;
                EngineParams p;
                base_params(&p, B, D, V, cdt, 0, 1, status);
                p.out = de32;
                p.ldo = D;
                p.out_dtype = CCE_DT_F32;
                p.accumulate = ps == 0 ? 0 : 2;  // the first pass stores every tile, later passes add with red
                p.sparse = 1;
                p.pass_info = pinfo;
                p.slot_tile = slot_tile;
                p.row_ptr = row_ptr;
                p.n_vt = pl.n_vt;
                p.klist = de_list;
                p.kcount = de_cnt;
                p.m_dev = ndev;
                set_peers(p);
                if (tile_ctr) p.tile_counter = tile_ctr + 4 * ps + 2;
                return run_de(p, tmP_k);
            };
            // in the last pass dE goes first when the caller wants to start reducing it early
            const bool de_first = early_de && ps == pl.max_pass - 1;
            rc = de_first ? pass_de() : pass_dc();
            if (rc != CCE_OK) return rc;
            if (de_first) {
                rc = finish_de();
                if (rc != CCE_OK) return rc;
            }
            rc = de_first ? pass_dc() : pass_de();
            if (rc != CCE_OK) return rc;
        }
    } else {
        uint8_t* flag_e = reinterpret_cast<uint8_t*>(ws + pl.off_flag_e);
        uint8_t* flag_c = reinterpret_cast<uint8_t*>(ws + pl.off_flag_c);
        for (int ch = 0; ch < pl.n_chunk; ++ch) {
            const long long v0 = (long long)ch * pl.Vc;
            const long long Vw = (V - v0 < pl.Vc) ? (V - v0) : pl.Vc;
            if (use_flags) CCE_CUDA(cudaMemsetAsync(flag_e, 0, pl.flag_bytes, st));

            // phase 1: G = dLoss/dLogits for columns [v0, v0 + Vw)
            {
                EngineParams p = pg;
                p.N = int(Vw);
                p.n_nblk = int(cdiv(Vw, BN));
                p.b_mn_off = int(v0);
                p.col_off = int(v0);
                p.ldg = pl.Vc;
                p.flag_e = flag_e;
                p.ld_flag_e = pl.ld_flag_e;
                p.flag_c = flag_c;
                p.ld_flag_c = pl.ld_flag_c;
                const bool pair = can_pair && p.n_mblk >= 2;
                rc = launch_engine<MODE_PGRAD>(tmE_k, pair ? tmC_k_h : tmC_k, p, dev->sms, st, pair);
                if (rc != CCE_OK) return rc;
            }

            // phase 2: dC[v0 : v0 + Vw, :] = G^T E   (M = Vw, N = D, K = B; both operands MN-major)
            auto chunk_dc = [&]() -> int {
                if (!a->d_c) return CCE_OK;
                CUtensorMap tmG_mn;
                int g_is3 = 0;  // the chunk's pitch (a multiple of 256) covers the last group of 64 columns
                rc = make_tmap_mn(&tmG_mn, g_buf, cdt, Vw, B, pl.Vc, BM / 64, tma3_enabled(), &g_is3);
                if (rc != CCE_OK) return rc;
                EngineParams p;
                base_params(&p, Vw, D, B, cdt, 1, 1, status);
                p.a_tma3 = g_is3;
                p.k_dev = ndev;
                p.out = reinterpret_cast<char*>(a->d_c) + (size_t)v0 * D * esz;
                p.ldo = D;
                p.out_dtype = split ? CCE_DT_F32 : op->dtype;
                p.accumulate = 0;
                if (a->has_filter && a->filter_c) {
                    p.kflags = flag_c;
                    p.ld_kflags = pl.ld_flag_c;
                }
                return run_dc(p, tmG_mn);
            };

            // phase 3: dE += G C[v0 : v0 + Vw, :]    (M = B, N = D, K = Vw; A K-major, B MN-major)
            auto chunk_de = [&]() -> int {
                if (!a->d_e) return CCE_OK;
                CUtensorMap tmG_k;
                rc = make_tmap(&tmG_k, g_buf, cdt, Vw, B, pl.Vc, BK, BM);
                if (rc != CCE_OK) return rc;
                EngineParams p;
                base_params(&p, B, D, Vw, cdt, 0, 1, status);
                p.b_k_off = int(v0);
                p.out = de32;
                p.ldo = D;
                p.out_dtype = CCE_DT_F32;
                p.accumulate = ch == 0 ? 0 : 2;  // the first chunk stores every tile, later chunks add with red
                p.m_dev = ndev;
                if (a->has_filter && a->filter_e) {
                    p.kflags = flag_e;
                    p.ld_kflags = pl.ld_flag_e;
                }
                set_peers(p);
                return run_de(p, tmG_k);
            };
            const bool de_first = early_de && ch == pl.n_chunk - 1;
            rc = de_first ? chunk_de() : chunk_dc();
            if (rc != CCE_OK) return rc;
            if (de_first) {
                rc = finish_de();
                if (rc != CCE_OK) return rc;
            }
            rc = de_first ? chunk_dc() : chunk_de();
            if (rc != CCE_OK) return rc;

            // bias gradient: column sums of G, partial sums per row block then a fixed-order finish
            if (a->d_bias) {
                const int n_rowblk = int(cdiv(B, kColsumRows));
                float* partial = reinterpret_cast<float*>(ws + pl.off_colsum);
                dim3 grid((unsigned)cdiv(Vw, 256), (unsigned)n_rowblk);
                if (cdt == CCE_DT_BF16)
                    colsum_partial_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(
                        reinterpret_cast<const __nv_bfloat16*>(g_buf), pl.Vc, B, int(Vw), kColsumRows, partial, pl.Vc, ndev);
                else
                    colsum_partial_kernel<__half><<<grid, 128, 0, st>>>(reinterpret_cast<const __half*>(g_buf), pl.Vc,
                                                                        B, int(Vw), kColsumRows, partial, pl.Vc, ndev);
                CCE_LAUNCH_CHECK();
                colsum_finish_kernel<<<(unsigned)cdiv(Vw, 256), 256, 0, st>>>(partial, pl.Vc, n_rowblk, int(Vw),
                                                                              a->d_bias + v0);
                CCE_LAUNCH_CHECK();
            }
        }
    }

    rc = finish_de();
    if (rc != CCE_OK) return rc;
    return CCE_OK;
}

int cce_b200_selftest_wait(int64_t limit_cycles, int32_t* status, void* stream) {
    if (!status || limit_cycles <= 0 || limit_cycles > 2000000000LL) return CCE_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    CCE_CUDA(cudaMemsetAsync(status, 0, 4, st));
    selftest_wait_kernel<<<1, 32, 0, st>>>((long long)limit_cycles, status);
    CCE_LAUNCH_CHECK();
    return CCE_OK;
}

int cce_b200_lse_forward_static_status(void* stream, int32_t* word) {
    void* scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc != CCE_OK) return rc;
    return cce_b200_read_status(scratch, stream, word);
}

int cce_b200_gemm(const void* A, const void* Bm, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                  int64_t ldb, int64_t ldo, int32_t dtype, int32_t out_dtype, int32_t a_mn, int32_t b_mn,
                  int32_t accumulate, const uint8_t* kflags, int32_t* status, void* stream) {
    if (!A || !Bm || !out || M <= 0 || N <= 0 || K <= 0) return CCE_ERR_ARG;
    if (dtype != CCE_DT_F16 && dtype != CCE_DT_BF16) return CCE_ERR_ARG;
    if (out_dtype != CCE_DT_F32 && out_dtype != dtype) return CCE_ERR_ARG;
    if (accumulate && out_dtype != CCE_DT_F32) return CCE_ERR_ARG;
    DeviceInfo* dev = nullptr;
    int rc = device_info(&dev);
    if (rc != CCE_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    CUtensorMap tmA, tmB;
    int a_is3 = 0, b_is3 = 0;
    if (!a_mn)
        rc = make_tmap(&tmA, A, dtype, K, M, lda, BK, BM);
    else
        rc = make_tmap_mn(&tmA, A, dtype, M, K, lda, BM / 64, tma3_enabled() && M % 64 == 0, &a_is3);
    if (rc != CCE_OK) return rc;
    // CTA pairs when nothing is skipped, two row blocks exist and MN-major operands have 3-D maps
    const bool pair = pair_enabled() && !kflags && M > BM && dev->sms >= 2 && (!a_mn || a_is3) &&
                      (!b_mn || (tma3_enabled() && N % 64 == 0));
    const int b_rows = pair ? BN / 2 : BN;  // rows of the B side each CTA stages
    if (!b_mn)
        rc = make_tmap(&tmB, Bm, dtype, K, N, ldb, BK, b_rows);
    else
        rc = make_tmap_mn(&tmB, Bm, dtype, N, K, ldb, b_rows / 64, tma3_enabled() && N % 64 == 0, &b_is3);
    if (rc != CCE_OK) return rc;
    if (pair && b_mn && !b_is3) return CCE_ERR_CUDA;  // the 3-D map the pair form needs was refused
    if (status) CCE_CUDA(cudaMemsetAsync(status, 0, 4, st));
    EngineParams p;
    base_params(&p, M, N, K, dtype, a_mn, b_mn, status);
    p.out = out;
    p.ldo = ldo;
    p.out_dtype = out_dtype;
    p.accumulate = accumulate;
    p.kflags = kflags;
    p.ld_kflags = int(cdiv(K, BK));
    p.a_tma3 = a_is3;
    p.b_tma3 = b_is3;
    return launch_engine<MODE_GEMM>(tmA, tmB, p, dev->sms, st, pair);
}

}  // extern "C"
