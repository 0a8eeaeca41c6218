// CTA-pair version of the tile kernels: a cluster of two CTAs computes one 256 x BN tile with
// tcgen05.mma.cta_group::2.  Each CTA stages only its own 128 rows of A and its own half of the
// B rows (BN/2), so every operand byte crosses L2 -> shared memory once per 256 x BN tile instead
// of once per 128 x BN tile, and a stage is 16 KiB + BN/2 * 128 B (6 stages at BN = 256).
//
// Roles per CTA (320 threads, as in umma_gemm.cuh):
//   warp 0  TMA producer for this CTA's halves; the byte count of both CTAs lands on the LEADER's
//           `full` barrier (rank 0 of the pair)
//   warp 1  TMEM allocation in both CTAs; the leader's lane 0 issues the MMAs for the pair and
//           releases stages / publishes accumulators in BOTH CTAs with multicast commits
//   warps 2-9  epilogue of this CTA's 128 accumulator rows (same three epilogues); the peer's
//           epilogue warps tell the leader that an accumulator is free with a remote arrive
// B is K-major here (the backward keeps transposed copies of X and Y); A is K-major or the
// column-blocked coefficient panel read as G (K-major) or G^T (MN-major).
// Tiles come from the same atomic counter as in the single-CTA kernel (strips included): the leader's
// scheduler lane fetches them and publishes each tile id into the ring of BOTH CTAs (a remote store followed by
// a remote release-arrive; the peer waits with a cluster-scope acquire).  A ring slot is free again when the
// consumers of both CTAs have arrived on the leader's `sched_empty` barrier (one arrive per warp).
// The last column tile of an output kernel may be narrower (bn_last), as in the single-CTA kernel.
#pragma once
#include <type_traits>

#include "umma_gemm.cuh"

namespace meclip {

static constexpr int PAIR_BM = 256;

// A_MODE: 0 = A is K-major, 1 = A is MN-major, 2 = two contractions in one launch (GemmParams::dual): the first
// problem reads A MN-major through tmap_a / tmap_b, the second one K-major through tmap_c (its A) / tmap_d (its B).
// TF32: A and B are fp32 matrices (both K-major) whose elements the tensor cores read as tf32; a K step is still
// 128 bytes per row (32 elements instead of 64), so stages, descriptors and barriers are those of the bf16 kernel.
template <int EPI, int A_MODE, bool TF32 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_d,
                      const __grid_constant__ GemmParams p) {
    constexpr bool DUAL = A_MODE == 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    const uint32_t stages_bytes = (uint32_t)p.num_stages * (uint32_t)p.stage_bytes;
    const uint32_t tail_off = ((stages_bytes + 1023u) & ~1023u) + (uint32_t)tail_bytes(EPI) - (uint32_t)sizeof(SharedTail);
    SharedTail* tail = reinterpret_cast<SharedTail*>(smem + (int)tail_off);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader of the pair
    const int num_tiles = DUAL ? p.tiles0 + p.num_m_tiles2 * p.num_n_tiles : p.num_m_tiles * p.num_n_tiles;
    const int num_clusters = (int)(gridDim.x >> 1);
    const int cluster_id = blockIdx.x >> 1;
    const int num_stages = p.num_stages;
    const int half_bn = p.bn >> 1;
    volatile int* abort_flag = &tail->abort_flag;
    const unsigned long long wl = p.wait_limit_ns;      // bound of every wait below (host-set, 2 s by default)

    if (threadIdx.x == 0) {
        tail->abort_flag = 0;
        for (int s = 0; s < num_stages; ++s) {
            mbar_init(smem_u32(&tail->full_bar[s]), 1);      // used in the leader only
            mbar_init(smem_u32(&tail->empty_bar[s]), 1);     // one multicast commit per use
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tail->tmem_full_bar[a]), 1);
            mbar_init(smem_u32(&tail->tmem_empty_bar[a]), 2 * EPI_WARPS);  // epilogue warps of both CTAs (leader only)
        }
        for (int s = 0; s < SCHED_DEPTH; ++s) {
            mbar_init(smem_u32(&tail->sched_full_bar[s]), 1);                   // the leader's scheduler arrives in both CTAs
            // leader only: its MMA lane and epilogue warps, the peer's producer lane and epilogue warps
            mbar_init(smem_u32(&tail->sched_empty_bar[s]), 2 + 2 * EPI_WARPS);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        if (EPI == EPI_COEF || DUAL) tma_prefetch_desc(&tmap_c);
        if (DUAL) tma_prefetch_desc(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tail->tmem_base), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- tile scheduler (leader) + TMA producer (both CTAs) ----------------
        if (lane == 0) {
            const uint32_t tx_per_cta = (uint32_t)A_STAGE_BYTES + (uint32_t)half_bn * BK * 2;
            int stage = 0, slot = 0;
            uint32_t phase = 0, sphase = 0;
            bool ok = true;
            // leader only: strips of consecutive tile ids, the next strip requested when one starts
            const int strip = p.strip_len;
            int unit = cluster_id;
            int next_tile = unit * strip;
            int left = strip;
            unsigned int next_unit = 0;
            while (ok) {
                int tile;
                if (rank == 0) {
                    if (!mbar_wait_cluster(smem_u32(&tail->sched_empty_bar[slot]), sphase ^ 1u, abort_flag, true, wl)) break;
                    tile = next_tile < num_tiles ? next_tile : -1;
                    tail->sched_tile[slot] = tile;
                    st_cluster_u32(mapa_u32(smem_u32(&tail->sched_tile[slot]), 1), (uint32_t)tile);
                    mbar_arrive(smem_u32(&tail->sched_full_bar[slot]));
                    mbar_arrive_cluster(mapa_u32(smem_u32(&tail->sched_full_bar[slot]), 1));
                    if (tile >= 0 && left == strip && p.tile_counter != nullptr)
                        asm volatile("atom.global.add.u32 %0, [%1], 1;" : "=r"(next_unit) : "l"(p.tile_counter) : "memory");
                } else {
                    if (!mbar_wait_cluster(smem_u32(&tail->sched_full_bar[slot]), sphase, abort_flag, true, wl)) break;
                    tile = tail->sched_tile[slot];
                    mbar_arrive_cluster(mapa_u32(smem_u32(&tail->sched_empty_bar[slot]), 0));
                }
                if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
                if (tile < 0) break;
                int mt, nt, t_rel = tile;
                const int prob = DUAL ? tile_problem(p, t_rel) : 0;
                tile_coords(p, t_rel, mt, nt, prob);
                const bool a_mn = DUAL ? prob == 0 : A_MODE == 1;
                const CUtensorMap* ta = (DUAL && prob == 1) ? &tmap_c : &tmap_a;
                const CUtensorMap* tb = (DUAL && prob == 1) ? &tmap_d : &tmap_b;
                const int k_steps = (DUAL && prob == 1) ? p.k_steps2 : p.k_steps;
                const int tile_bn = (nt == p.num_n_tiles - 1) ? p.bn_last : p.bn;
                const int m0 = mt * PAIR_BM + (int)rank * BM;              // this CTA's rows
                const int n0 = nt * p.bn + (int)rank * (tile_bn >> 1);      // this CTA's share of the B rows
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait(smem_u32(&tail->empty_bar[stage]), phase ^ 1u, abort_flag, true, wl)) { ok = false; break; }
                    const uint32_t full_local = smem_u32(&tail->full_bar[stage]);
                    const uint32_t full = mapa_u32(full_local, 0);    // the leader's barrier counts both CTAs' bytes
                    if (rank == 0) mbar_expect_tx(full_local, 2u * tx_per_cta);
                    const uint32_t sa = smem_base + (uint32_t)stage * (uint32_t)p.stage_bytes;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const int k0 = ks * (TF32 ? BK / 2 : BK);       // in elements
                    if (p.a_blocked) {
                        if (a_mn) {
                            tma_load_3d_pair(sa, ta, full, 0, k0, m0 >> 6);
                            tma_load_3d_pair(sa + BK * 128, ta, full, 0, k0, (m0 >> 6) + 1);
                        } else {
                            tma_load_3d_pair(sa, ta, full, 0, m0, ks);
                        }
                    } else if (a_mn) {
                        tma_load_2d_pair(sa, ta, full, m0, k0);
                        tma_load_2d_pair(sa + BK * 128, ta, full, m0 + 64, k0);
                    } else {
                        tma_load_2d_pair(sa, ta, full, k0, m0);
                    }
                    // the box always has half_bn rows; a narrower last tile uses the first tile_bn / 2 of them
                    tma_load_2d_pair(sb, tb, full, k0, n0);
                    if (++stage == num_stages) { stage = 0; phase ^= 1u; }
                }
                if (rank == 0) {
                    if (--left > 0 && next_tile + 1 < num_tiles) {
                        ++next_tile;
                    } else {
                        unit = p.tile_counter != nullptr ? (int)next_unit + num_clusters : unit + num_clusters;
                        next_tile = unit * strip;
                        left = strip;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ---------------
        if (lane == 0 && rank == 0) {
            int stage = 0, slot = 0;
            uint32_t phase = 0, sphase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            while (ok) {
                if (!mbar_wait(smem_u32(&tail->sched_full_bar[slot]), sphase, abort_flag, true, wl)) break;
                const int tile = tail->sched_tile[slot];
                mbar_arrive(smem_u32(&tail->sched_empty_bar[slot]));
                if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
                if (tile < 0) break;
                if (!mbar_wait_cluster(smem_u32(&tail->tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag, true, wl)) break;
                tc_fence_after();
                int mt_, nt_, t_rel = tile;
                const int prob = DUAL ? tile_problem(p, t_rel) : 0;
                tile_coords(p, t_rel, mt_, nt_, prob);
                const bool a_mn = DUAL ? prob == 0 : A_MODE == 1;
                const int k_steps = (DUAL && prob == 1) ? p.k_steps2 : p.k_steps;
                const bool last_nt = nt_ == p.num_n_tiles - 1;
                const uint32_t idesc = (DUAL && prob == 1) ? (last_nt ? p.idesc_last_p2 : p.idesc_p2)
                                                           : (last_nt ? p.idesc_last : p.idesc);
                const uint32_t idesc2 = last_nt ? p.idesc2_last : p.idesc2;       // second MMA of a wide tile
                const int tile_bn_ = last_nt ? p.bn_last : p.bn;
                // rows of this CTA's B half that the first MMA consumes; the second one starts behind them
                const uint32_t b2_off = (uint32_t)(min(tile_bn_, MAX_BN) >> 1) * 128u;
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * MAX_BN;
                // The K loop with A's majorness as a compile-time constant: the issuing thread's instruction stream
                // per K step decides how well the tensor pipe is fed, so the dual launch gets one copy of the loop per
                // majorness instead of run-time descriptor strides.
                auto k_loop = [&](auto amn_tag) -> bool {
                    constexpr bool AMN = decltype(amn_tag)::value;
                    constexpr uint32_t A_LBO = AMN ? BK * 128 : 16, A_KSTEP = AMN ? 2048 : 32;
                    for (int ks = 0; ks < k_steps; ++ks) {
                        if (!mbar_wait(smem_u32(&tail->full_bar[stage]), phase, abort_flag, true, wl)) return false;
                        tc_fence_after();
                        const uint32_t sa = smem_base + (uint32_t)stage * (uint32_t)p.stage_bytes;
                        const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk) {
                            const uint64_t ad = umma_smem_desc(sa + kk * A_KSTEP, A_LBO, 1024);
                            const uint64_t bd = umma_smem_desc(sb + kk * 32, 16, 1024);
                            if (TF32) umma_tf32_pair(tmem_d, ad, bd, idesc, (ks | kk) != 0 ? 1u : 0u);
                            else      umma_bf16_pair(tmem_d, ad, bd, idesc, (ks | kk) != 0 ? 1u : 0u);
                            if (idesc2 != 0u) {
                                const uint64_t bd2 = umma_smem_desc(sb + b2_off + kk * 32, 16, 1024);
                                umma_bf16_pair(tmem_d + MAX_BN, ad, bd2, idesc2, (ks | kk) != 0 ? 1u : 0u);
                            }
                        }
                        umma_commit_pair(smem_u32(&tail->empty_bar[stage]), 3);     // frees the stage in both CTAs
                        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
                    }
                    return true;
                };
                if (DUAL) ok = a_mn ? k_loop(std::true_type{}) : k_loop(std::false_type{});
                else      ok = k_loop(std::integral_constant<bool, A_MODE == 1>{});
                if (!ok) break;
                umma_commit_pair(smem_u32(&tail->tmem_full_bar[acc]), 3);       // accumulator halves complete
                if (p.wide) {
                    acc_phase ^= 1u;             // one accumulator of up to 512 columns: every tile flips its phase
                } else {
                    acc ^= 1;
                    if (acc == 0) acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;
        int acc = 0, slot = 0;
        uint32_t acc_phase = 0, sphase = 0;
        EpiState st;
        epilogue_init<EPI>(p, st);
        const uint32_t sched_free0 = mapa_u32(smem_u32(&tail->sched_empty_bar[0]), 0);     // the leader's ring
        while (true) {
            // as in the single-CTA kernel the eight warps reach one decision per wait and leave together
            bool ok = mbar_wait_cluster(smem_u32(&tail->sched_full_bar[slot]), sphase, abort_flag, false, wl);
            const int tile = ok ? tail->sched_tile[slot] : -1;
            __syncwarp();
            if (ok && lane == 0) mbar_arrive_cluster(sched_free0 + (uint32_t)slot * 8u);
            if (++slot == SCHED_DEPTH) { slot = 0; sphase ^= 1u; }
            ok = named_bar_and(2, EPI_THREADS, ok);
            if (!ok || tile < 0) break;
            int mt, nt, t_rel = tile;
            const int prob = DUAL ? tile_problem(p, t_rel) : 0;
            tile_coords(p, t_rel, mt, nt, prob);
            ok = mbar_wait(smem_u32(&tail->tmem_full_bar[acc]), acc_phase, abort_flag, false, wl);
            ok = named_bar_and(2, EPI_THREADS, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * MAX_BN;
            const uint32_t free_bar = mapa_u32(smem_u32(&tail->tmem_empty_bar[acc]), 0);   // the leader's barrier
            epilogue_tile<EPI>(p, out_desc(p, prob), &tmap_c, tail, st, taddr, mt * PAIR_BM + (int)rank * BM, nt * p.bn,
                               (nt == p.num_n_tiles - 1) ? p.bn_last : p.bn, warp, lane,
                               [free_bar, lane]() {
                                   __syncwarp();
                                   if (lane == 0) mbar_arrive_cluster(free_bar);
                               });
            if (p.wide) {
                acc_phase ^= 1u;
            } else {
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
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
            const unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 2000000ull) { __nanosleep(1000); }
        }
        __syncthreads();
    }
    // neither CTA may leave while the other can still read its shared memory or signal its barriers
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace meclip
