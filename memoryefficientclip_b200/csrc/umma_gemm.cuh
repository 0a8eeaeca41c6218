// Persistent, warp-specialised tcgen05 GEMM mainloop shared by every tile kernel
// of the loss path, with three epilogues:
//
//   EPI_SUMS  S = X Y^T tile -> E = exp2(k S - k) -> row sums, column sums, diagonal
//   EPI_COEF  S tile -> E -> G = E (g/r_i + g/c_j) - [i==j] g -> bf16 panel, TMA-stored in a
//             column-blocked layout [64-column chunk][row][64] so that every later tile load of
//             the panel (as G or as G^T) is one contiguous run of memory
//   EPI_OUT   plain contraction -> (+ fp32 partial) -> fp32 / bf16 store
//
// One CTA per SM, 320 threads:
//   warp 0      tile scheduler + TMA producer (one lane): global -> 128B-swizzled shared tiles
//   warp 1      TMEM allocator + MMA issuer (one lane): tcgen05.mma 128 x BN x 16, bf16 -> fp32
//   warps 2-9   epilogue (epilogue.cuh): tcgen05.ld of the finished accumulator while the MMA
//               warp already fills the other accumulator (2 x 256 TMEM columns)
// Tiles are handed out dynamically (one atomic per tile on a caller-zeroed counter) when a
// counter is given, so that kernels sharing the GPU with each other balance themselves;
// without a counter the tiles are dealt round-robin.
// A and B operands may each be K-major (K contiguous in global memory) or MN-major
// (M / N contiguous), so G, G^T, X and Y are all consumed from their one row-major copy.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace meclip {

static constexpr int BM = 128;            // tile rows  (UMMA M)
static constexpr int BK = 64;             // K per stage: 64 bf16 = one 128-byte swizzle row
static constexpr int MAX_BN = 256;        // tile columns (UMMA N), runtime value <= this
static constexpr int MAX_STAGES = 8;
static constexpr int SCHED_DEPTH = 4;     // tile ids in flight between the scheduler and the consumers
static constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KiB
static constexpr int TMEM_COLS = 512;     // two accumulators of up to 256 columns
// Build-time shape of the epilogue: 4 or 8 warps, and whether the sums pass keeps its column partials in
// registers over a strip of tiles (needs 8 warps: 128 accumulators per thread) or reduces them per tile.
#ifndef MECLIP_EPI_WARPS
#define MECLIP_EPI_WARPS 8
#endif
#ifndef MECLIP_STRIPS
#define MECLIP_STRIPS (MECLIP_EPI_WARPS == 8)
#endif
static constexpr int EPI_WARPS = MECLIP_EPI_WARPS;
static constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;   // producer warp + MMA warp + epilogue warps
static constexpr int EPI_THREADS = 32 * EPI_WARPS;
static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "4 or 8 epilogue warps");
static_assert(!MECLIP_STRIPS || EPI_WARPS == 8, "strip accumulators need 8 epilogue warps");
static constexpr int SMEM_LIMIT = 232448; // 227 KiB: most dynamic shared memory one CTA can have
static constexpr int STORE_BUF_BYTES = 32 * 128;   // one warp's 32 rows x 64 bf16 staging tile

enum { EPI_SUMS = 0, EPI_COEF = 1, EPI_OUT = 2 };

struct GemmParams {
    int m, n, k;              // valid extents of the problem
    int bn;                   // tile width (multiple of 32; multiple of 64 when B is MN-major)
    int num_m_tiles, num_n_tiles, k_steps;
    int group_m;              // rasterisation: m-tiles per group swept along n
    int num_stages;           // operand ring depth, from the shared memory left over
    int stage_bytes;          // A_STAGE_BYTES + bn * 128
    uint32_t idesc;
    // The last column tile may be narrower (EPI_OUT only): 1152 columns = 4 tiles of 256 + one of 128, which
    // feeds the tensor cores better than six tiles of 192.  bn_last == bn when there is no such tile.
    int bn_last;
    uint32_t idesc_last;
    // Wide tiles (CTA-pair kernel, EPI_OUT only): bn in (256, 512].  A tile is then computed by TWO MMAs per K
    // step that share the A operand in shared memory (N = 256 into TMEM columns 0.., N = bn - 256 into columns
    // 256..), and the one 512-column accumulator is not double-buffered: with K in the thousands the epilogue
    // is ~1 % of a tile.  Operand bytes per FLOP drop by 17 % (bn = 384) / 25 % (bn = 512) against 256 x 256.
    int wide;
    uint32_t idesc2, idesc2_last;   // second MMA of a wide tile (0: none)
    unsigned int* tile_counter;   // zeroed by the caller; null = static round-robin
    int strip_len;            // tiles handed out together (consecutive ids share their columns), >= 1
    int a_blocked;            // A is the coefficient panel in its column-blocked layout (3-D tensor map)
    // EPI_SUMS / EPI_COEF
    // The elementwise function of the similarity s is f(fmul * s + fadd):
    //   softmax losses (CLIP, LiT): f = exp2, fmul = log2(e)/T, fadd = -log2(e)/T
    //   sigmoid loss: fmul = t log2(e), fadd = b log2(e); SUMS f = softplus in base-2 units,
    //                 COEF f = sigmoid = 1 / (1 + 2^-u)
    float fmul, fadd;
    int sigmoid;              // 0 = exp2, 1 = the sigmoid-loss functions
    long long diag_shift;     // (row_off - col_off): row i meets column i + diag_shift
    float* row_sum;           // SUMS: accumulated with atomics
    float* col_sum;           // SUMS: may be null (LiT)
    float* diag;              // SUMS: S_ii per row, written where the diagonal crosses the block
    // SUMS, deterministic mode: instead of atomics every partial sum is STORED in its own slot and a second kernel
    // adds the slots in a fixed order.  row_part[(2 * column tile + warp group) * part_ld_rows + row],
    // col_part[(row / 128) * part_ld_cols + column]; both null = atomics.
    float* row_part;
    float* col_part;
    long long part_ld_rows, part_ld_cols;
    const float* r;           // COEF: saved row sums
    const float* c;           // COEF: saved column sums or null (LiT)
    const float* grad_out;    // COEF: device scalar
    float coef;               // COEF: grad_scale * (0.5 for CLIP, 1 for LiT)
    float dcoef;              // COEF: grad_scale (subtracted on the diagonal)
    float* sg_acc;            // COEF: optional, [0] += sum_ij G_ij S_ij, [1] += sum_ij G_ij (fp32 G before rounding)
    // EPI_OUT
    void* out;
    long long ld_out;
    int out_bf16;
    const float* acc_in;      // optional fp32 partial added before the store
    long long ld_acc;
    // Two contractions in ONE launch (CTA-pair kernel, EPI_OUT, A_MODE = 2): tile ids below tiles0 belong to the first
    // problem (the fields above; its A is read MN-major: dY = G^T X), the others to the second one (dX = G Y, A read
    // K-major).  Both share n, bn and the tile width of the last column tile; rows, K, outputs and the instruction
    // descriptors (they carry A's majorness) are per problem.  One launch of 640 tiles ends in a fuller last wave
    // than two launches of 320 (74 CTA pairs).
    int dual, tiles0;
    int m2, k_steps2, num_m_tiles2;
    uint32_t idesc_p2, idesc_last_p2;
    void* out2;
    long long ld_out2;
    int out_bf16_2;
    const float* acc_in2;
    long long ld_acc2;
    int* status;
    unsigned long long wait_limit_ns;   // bound of every barrier wait inside the kernel
    // Scalars that live on the device (a learnable temperature / logit scale / bias): when t_dev is set the
    // epilogues derive fmul / fadd from it instead of using the host values above, and the coefficient scale
    // g = coef * (*grad_out) is multiplied by a power of it (g_rule: 0 none, 1 1/T, 2 1/sqrt(T), 3 t).
    const float* t_dev;
    const float* b_dev;       // sigmoid loss: logit bias on the device (null: fadd as given)
    int g_rule;
    // EPI_OUT with a narrower last column tile: hand out all full-width tiles first and the narrow ones last,
    // so that the short tiles fill the end of the launch (longest-processing-time order)
    int narrow_last;
    // Optional in-kernel trace (test hook): CTA 0 appends {tag, tile, %globaltimer} records.
    // Records of 3 words start at trace[2]; role r owns records [r*cap/3, (r+1)*cap/3); unused ones stay zero.
    unsigned long long* trace;
    unsigned int trace_capacity;
};

enum { TR_LOAD_BEGIN = 1, TR_LOAD_END = 2, TR_MMA_BEGIN = 10, TR_MMA_FIRST_DATA = 11, TR_MMA_END = 12,
       TR_EPI_BEGIN = 20, TR_EPI_RELEASED = 21, TR_EPI_END = 22 };

// Each role (0 producer, 1 MMA issuer, 2 epilogue) appends to its own third of the buffer with a
// private counter, so a record is three plain stores and does not wait on memory.
__device__ __forceinline__ void trace_event(const GemmParams& p, int role, unsigned int& count, int tag, int tile) {
    if (p.trace == nullptr || blockIdx.x != 0) return;
    const unsigned int per_role = p.trace_capacity / 3;
    if (count < per_role) {
        unsigned long long* rec = p.trace + 2 + 3ull * ((unsigned long long)role * per_role + count);
        rec[0] = (unsigned long long)tag;
        rec[1] = (unsigned long long)(long long)tile;
        rec[2] = global_ns();
        ++count;
    }
}

// Everything in shared memory that is not an operand stage.  `scratch` is a union by use:
// SUMS keeps per-quadrant column partials there (4 x 256 floats), COEF its TMA-store staging
// tiles (8 warps x 4 KiB, 1024-byte aligned for the 128-byte swizzle).
struct SharedTail {
    uint8_t scratch[4 * 2 * STORE_BUF_BYTES];   // placed on a 1024-byte boundary by the kernel
    float icol[MAX_BN];         // COEF: g / c_j for the tile's columns
    unsigned long long full_bar[MAX_STAGES];
    unsigned long long empty_bar[MAX_STAGES];
    unsigned long long tmem_full_bar[2];
    unsigned long long tmem_empty_bar[2];
    unsigned long long sched_full_bar[SCHED_DEPTH];
    unsigned long long sched_empty_bar[SCHED_DEPTH];
    int sched_tile[SCHED_DEPTH];
    uint32_t tmem_base;
    int abort_flag;
};

__host__ __device__ constexpr int tail_bytes(int epi) {
    // the scratch union is the first member; kernels that do not need all of it start the tail later
    return (int)sizeof(SharedTail) - (epi == EPI_COEF ? 0 : epi == EPI_SUMS ? 4 * 2 * STORE_BUF_BYTES - 4 * MAX_BN * 4
                                                                            : 4 * 2 * STORE_BUF_BYTES);
}

template <int HALF>
__device__ __forceinline__ void transpose_reduce_step(float (&v)[32], int lane) {
    const bool up = (lane & HALF) != 0;
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
        const float send = up ? v[i] : v[i + HALF];
        const float keep = up ? v[i + HALF] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, HALF);
    }
}
// Sum over the warp of v[slot] for each of 32 slots: lane L returns the total of slot L.
// 31 shuffles instead of 32 x 5.
__device__ __forceinline__ float warp_transpose_reduce32(float (&v)[32], int lane) {
    transpose_reduce_step<16>(v, lane);
    transpose_reduce_step<8>(v, lane);
    transpose_reduce_step<4>(v, lane);
    transpose_reduce_step<2>(v, lane);
    transpose_reduce_step<1>(v, lane);
    return v[0];
}

// What the plain-contraction epilogue needs to know about the problem a tile belongs to.
struct OutDesc {
    int m;                    // valid rows
    void* out;
    long long ld_out;
    int out_bf16;
    const float* acc_in;
    long long ld_acc;
};

// Problem of a tile id in a dual launch (0 or 1); the id is made relative to its problem.
__device__ __forceinline__ int tile_problem(const GemmParams& p, int& tile) {
    if (p.dual && tile >= p.tiles0) { tile -= p.tiles0; return 1; }
    return 0;
}
__device__ __forceinline__ OutDesc out_desc(const GemmParams& p, int problem) {
    if (problem == 0) return OutDesc{p.m, p.out, p.ld_out, p.out_bf16, p.acc_in, p.ld_acc};
    return OutDesc{p.m2, p.out2, p.ld_out2, p.out_bf16_2, p.acc_in2, p.ld_acc2};
}

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& mt, int& nt, int problem = 0) {
    const int num_m_tiles = problem == 0 ? p.num_m_tiles : p.num_m_tiles2;
    int n_tiles = p.num_n_tiles;
    if (p.narrow_last) {
        // ids [0, m_tiles * (n_tiles - 1)) walk the full-width column tiles in groups as below,
        // the remaining m_tiles ids are the narrow last column tile of every row tile
        n_tiles = p.num_n_tiles - 1;
        const int full = num_m_tiles * n_tiles;
        if (tile >= full) { mt = tile - full; nt = n_tiles; return; }
    }
    const int per_group = p.group_m * n_tiles;
    const int grp = tile / per_group;
    const int first_m = grp * p.group_m;
    const int rows_in_group = min(p.group_m, num_m_tiles - first_m);
    const int local = tile - grp * per_group;
    mt = first_m + local % rows_in_group;
    nt = local / rows_in_group;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace meclip
#include "epilogue.cuh"
namespace meclip {

template <int EPI, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    // The tail sits behind the stages; its unused leading part of `scratch` overlaps the last stage
    // region on purpose for SUMS / OUT (they never touch those bytes), see tail_bytes().
    const uint32_t stages_bytes = (uint32_t)p.num_stages * (uint32_t)p.stage_bytes;
    const uint32_t tail_off = ((stages_bytes + 1023u) & ~1023u) + (uint32_t)tail_bytes(EPI) - (uint32_t)sizeof(SharedTail);
    SharedTail* tail = reinterpret_cast<SharedTail*>(smem + (int)tail_off);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.num_m_tiles * p.num_n_tiles;
    const int num_stages = p.num_stages;
    volatile int* abort_flag = &tail->abort_flag;
    const unsigned long long wl = p.wait_limit_ns;      // bound of every wait below (host-set, 2 s by default)

    if (threadIdx.x == 0) {
        tail->abort_flag = 0;
        for (int s = 0; s < num_stages; ++s) {
            mbar_init(smem_u32(&tail->full_bar[s]), 1);
            mbar_init(smem_u32(&tail->empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tail->tmem_full_bar[a]), 1);
            mbar_init(smem_u32(&tail->tmem_empty_bar[a]), EPI_THREADS);
        }
        for (int s = 0; s < SCHED_DEPTH; ++s) {
            mbar_init(smem_u32(&tail->sched_full_bar[s]), 1);
            mbar_init(smem_u32(&tail->sched_empty_bar[s]), 1 + EPI_THREADS);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        if (EPI == EPI_COEF) tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ------------------- tile scheduler + TMA producer -------------------------
        if (lane == 0) {
            const uint32_t stage_tx = (uint32_t)A_STAGE_BYTES + (uint32_t)p.bn * BK * 2;
            int stage = 0, slot = 0;
            uint32_t phase = 0, sphase = 0;
            // Work is handed out in strips of strip_len consecutive tile ids (same columns, next rows):
            // the first strip is blockIdx.x, later ones come from the counter.  The next strip's id is
            // requested (one atomic, ~1 us round trip) when a strip STARTS and only read when it ends,
            // so the operand pipeline never waits for it.
            const int strip = p.strip_len;
            int unit = blockIdx.x;
            int tile = unit * strip;
            int left = strip;
            unsigned int next_unit = 0;
            unsigned int ntrace = 0;
            bool ok = true;
            while (ok) {
                // publish the tile id (or -1 = no more work) to the MMA and epilogue roles
                if (!mbar_wait(smem_u32(&tail->sched_empty_bar[slot]), sphase ^ 1u, abort_flag, true, wl)) break;
                const int pub = tile < num_tiles ? tile : -1;
                tail->sched_tile[slot] = pub;
                mbar_arrive(smem_u32(&tail->sched_full_bar[slot]));
                if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
                if (pub < 0) break;
                // First tile of a strip: ask for the strip after this one now.  next_unit is written by
                // nothing but the atomic, so nothing waits for its round trip before the strip ends.
                if (left == strip && p.tile_counter != nullptr)
                    asm volatile("atom.global.add.u32 %0, [%1], 1;" : "=r"(next_unit) : "l"(p.tile_counter) : "memory");
                int mt, nt;
                tile_coords(p, tile, mt, nt);
                const int m0 = mt * BM, n0 = nt * p.bn;
                trace_event(p, 0, ntrace, TR_LOAD_BEGIN, tile);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    if (!mbar_wait(smem_u32(&tail->empty_bar[stage]), phase ^ 1u, abort_flag, true, wl)) { ok = false; break; }
                    const uint32_t full = smem_u32(&tail->full_bar[stage]);
                    mbar_expect_tx(full, stage_tx);
                    const uint32_t sa = smem_base + (uint32_t)stage * (uint32_t)p.stage_bytes;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const int k0 = ks * BK;
                    if (p.a_blocked) {
                        // coefficient panel stored as [64-column chunk][row][64]: every box is one contiguous run
                        if (A_MN) {   // A = G^T: M runs along the panel's columns, K along its rows
                            tma_load_3d(sa, &tmap_a, full, 0, k0, m0 >> 6);
                            tma_load_3d(sa + BK * 128, &tmap_a, full, 0, k0, (m0 >> 6) + 1);
                        } else {      // A = G: M along rows, K along columns
                            tma_load_3d(sa, &tmap_a, full, 0, m0, ks);
                        }
                    } else if (A_MN) {   // global [K rows][M contiguous]: 64-wide column chunks of BK rows
                        tma_load_2d(sa, &tmap_a, full, m0, k0);
                        tma_load_2d(sa + BK * 128, &tmap_a, full, m0 + 64, k0);
                    } else {      // global [M rows][K contiguous]
                        tma_load_2d(sa, &tmap_a, full, k0, m0);
                    }
                    if (B_MN) {
                        for (int c = 0; c < p.bn / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmap_b, full, n0 + c * 64, k0);
                    } else {
                        tma_load_2d(sb, &tmap_b, full, k0, n0);
                    }
                    if (++stage == num_stages) { stage = 0; phase ^= 1u; }
                }
                trace_event(p, 0, ntrace, TR_LOAD_END, tile);
                if (--left > 0 && tile + 1 < num_tiles) {
                    ++tile;
                } else {
                    unit = p.tile_counter != nullptr ? (int)(next_unit + gridDim.x) : unit + (int)gridDim.x;
                    tile = unit * strip;
                    left = strip;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int stage = 0, slot = 0;
            uint32_t phase = 0, sphase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            unsigned int ntrace = 0;
            bool ok = true;
            // K-major: 8-row groups 1024 B apart (SBO), 32 B per K=16 step inside the swizzle row.
            // MN-major: 64-element chunks BK*128 B apart (LBO), 8-row K groups 1024 B apart (SBO),
            //           a K=16 step is 16 rows = 2048 B.
            constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, A_KSTEP = A_MN ? 2048 : 32;
            constexpr uint32_t B_LBO = B_MN ? BK * 128 : 16, B_KSTEP = B_MN ? 2048 : 32;
            while (ok) {
                if (!mbar_wait(smem_u32(&tail->sched_full_bar[slot]), sphase, abort_flag, true, wl)) break;
                const int tile = tail->sched_tile[slot];
                mbar_arrive(smem_u32(&tail->sched_empty_bar[slot]));
                if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
                if (tile < 0) break;
                if (!mbar_wait(smem_u32(&tail->tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag, true, wl)) break;
                tc_fence_after();
                trace_event(p, 1, ntrace, TR_MMA_BEGIN, tile);
                int mt_, nt_;
                tile_coords(p, tile, mt_, nt_);
                const uint32_t idesc = (nt_ == p.num_n_tiles - 1) ? p.idesc_last : p.idesc;
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * MAX_BN;
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    if (!mbar_wait(smem_u32(&tail->full_bar[stage]), phase, abort_flag, true, wl)) { ok = false; break; }
                    tc_fence_after();
                    if (ks == 0) trace_event(p, 1, ntrace, TR_MMA_FIRST_DATA, tile);
                    const uint32_t sa = smem_base + (uint32_t)stage * (uint32_t)p.stage_bytes;
                    const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t ad = umma_smem_desc(sa + kk * A_KSTEP, A_LBO, 1024);
                        const uint64_t bd = umma_smem_desc(sb + kk * B_KSTEP, B_LBO, 1024);
                        umma_bf16(tmem_d, ad, bd, idesc, (ks | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&tail->empty_bar[stage]));   // frees the stage when these MMAs retire
                    if (++stage == num_stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&tail->tmem_full_bar[acc]));     // accumulator complete
                trace_event(p, 1, ntrace, TR_MMA_END, tile);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;                 // TMEM lane quadrant this warp can read
        int acc = 0, slot = 0;
        uint32_t acc_phase = 0, sphase = 0;
        EpiState st;
        unsigned int ntrace = 0;
        epilogue_init<EPI>(p, st);
        while (true) {
            // The eight warps wait on the same barrier phase and then agree on the outcome, so that
            // they always leave the tile loop (and its named barriers) together.
            bool ok = mbar_wait(smem_u32(&tail->sched_full_bar[slot]), sphase, abort_flag, false, wl);
            int tile = -1;
            if (ok) {
                tile = tail->sched_tile[slot];
                mbar_arrive(smem_u32(&tail->sched_empty_bar[slot]));
            }
            if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
            ok = named_bar_and(2, EPI_THREADS, ok);
            if (!ok || tile < 0) break;
            int mt, nt;
            tile_coords(p, tile, mt, nt);
            ok = mbar_wait(smem_u32(&tail->tmem_full_bar[acc]), acc_phase, abort_flag, false, wl);
            ok = named_bar_and(2, EPI_THREADS, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * MAX_BN;
            const uint32_t free_bar = smem_u32(&tail->tmem_empty_bar[acc]);
            if (threadIdx.x == 64) trace_event(p, 2, ntrace, TR_EPI_BEGIN, tile);
            epilogue_tile<EPI>(p, out_desc(p, 0), &tmap_c, tail, st, taddr, mt * BM, nt * p.bn,
                               (nt == p.num_n_tiles - 1) ? p.bn_last : p.bn, warp, lane,
                               [free_bar, &p, &ntrace, tile]() {
                                   mbar_arrive(free_bar);
                                   if (threadIdx.x == 64) trace_event(p, 2, ntrace, TR_EPI_RELEASED, tile);
                               });
            if (threadIdx.x == 64) trace_event(p, 2, ntrace, TR_EPI_END, tile);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (EPI == EPI_SUMS && !tail->abort_flag) flush_column_sums(p, tail, st, warp, lane);
        epilogue_drain<EPI>(st, lane);
    }

    // ------------------------------ teardown ---------------------------------------
    tc_fence_before();
    __syncthreads();
    if (tail->abort_flag) {
        if (threadIdx.x == 0) {
            if (p.status != nullptr) atomicExch(p.status, 1);
            // give tile copies that may still be in flight time to land before the CTA's
            // shared memory is handed to another CTA
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 2000000ull) { __nanosleep(1000); }
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace meclip
