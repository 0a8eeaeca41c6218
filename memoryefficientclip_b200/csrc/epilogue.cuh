// The three epilogues of the tile kernels, shared by the single-CTA and the CTA-pair kernel.
// Eight warps (two per TMEM lane quadrant) work on one 128-row accumulator: warp quadrant
// q = warp % 4 owns rows 32q..32q+31, warp group wg = 0/1 owns the first / second half of the
// tile's columns.  One thread = one row (tcgen05.ld 32x32b), 32 columns per load.
#pragma once
#include "sm100_ptx.cuh"

namespace meclip {

struct EpiState {        // per-thread state that lives across tiles
    int stores_in_flight = 0;   // COEF: lane 0's outstanding TMA-store groups
    float gscale = 1.f;         // COEF: *grad_out
};

// `release()` is called by every thread once its last tcgen05.ld of the tile has completed; it must
// tell the MMA issuer that this thread is done with the accumulator.
template <int EPI, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const CUtensorMap* tmap_c, SharedTail* tail,
                                              EpiState& st, uint32_t taddr, int m0, int n0, int warp, int lane,
                                              Release release) {
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int et = (int)threadIdx.x - 64;                 // 0..255 within the epilogue group
    const int grow = m0 + q * 32 + lane;
    const bool rvalid = grow < p.m;
    const bool full_tile = (m0 + BM <= p.m) && (n0 + p.bn <= p.n);
    // column (tile-local) on which this row meets the diagonal, -1 if outside the tile
    const long long jd_ll = (long long)grow + p.diag_shift - n0;
    const int jd = (jd_ll >= 0 && jd_ll < p.bn && n0 + jd_ll < p.n && rvalid) ? (int)jd_ll : -1;
    // this warp group's share of the columns, in units of 32 (SUMS, OUT) or 64 (COEF) columns
    const int units = (EPI == EPI_COEF) ? (p.bn >> 6) : (p.bn >> 5);
    const int u_split = (units + 1) >> 1;
    const int u_begin = wg == 0 ? 0 : u_split;
    const int u_end = wg == 0 ? u_split : units;

    if (EPI == EPI_SUMS) {
        float (*colpart)[MAX_BN] = reinterpret_cast<float (*)[MAX_BN]>(tail->scratch + sizeof(tail->scratch) - 4 * MAX_BN * 4);
        float ra0 = 0.f, ra1 = 0.f, ra2 = 0.f, ra3 = 0.f;
        float sdiag = 0.f;
        for (int ch = u_begin; ch < u_end; ++ch) {
            uint32_t v[32];
            tmem_ld32(taddr + ch * 32, v);
            tmem_ld_wait();
            float e[32];
            const int jdc = (jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float sv = __uint_as_float(v[c]);
                e[c] = ex2_approx(fmaf(sv, p.k2, -p.k2));
                sdiag = (c == jdc) ? sv : sdiag;
            }
            if (!full_tile) {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (!rvalid || n0 + ch * 32 + c >= p.n) e[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 32; c += 4) { ra0 += e[c]; ra1 += e[c + 1]; ra2 += e[c + 2]; ra3 += e[c + 3]; }
            if (p.col_sum != nullptr) {
                const float cs = warp_transpose_reduce32(e, lane);
                colpart[q][ch * 32 + lane] = cs;
            }
        }
        tc_fence_before();
        release();
        if (rvalid && u_end > u_begin) atomicAdd(p.row_sum + grow, (ra0 + ra1) + (ra2 + ra3));
        if (jd >= 0 && (jd >> 5) >= u_begin && (jd >> 5) < u_end) p.diag[grow] = sdiag;
        if (p.col_sum != nullptr) {
            named_bar_sync(1, EPI_THREADS);
            for (int j = et; j < p.bn; j += EPI_THREADS)
                if (n0 + j < p.n)
                    atomicAdd(p.col_sum + n0 + j, (colpart[0][j] + colpart[1][j]) + (colpart[2][j] + colpart[3][j]));
            named_bar_sync(1, EPI_THREADS);
        }
    } else if (EPI == EPI_COEF) {
        // g / c_j for the tile's columns, staged once per tile for all eight warps
        named_bar_sync(1, EPI_THREADS);            // previous tile's readers of icol are done
        for (int j = et; j < p.bn; j += EPI_THREADS) {
            float v = 0.f;
            if (p.c != nullptr && n0 + j < p.n) v = p.coef * st.gscale / __ldg(p.c + n0 + j);
            tail->icol[j] = v;
        }
        const float inv_r = rvalid ? p.coef * st.gscale / __ldg(p.r + grow) : 0.f;
        named_bar_sync(1, EPI_THREADS);
        // Each warp turns 32 rows x 64 columns into a 128-byte-swizzled shared tile and one lane
        // TMA-stores it (full 128-byte lines; rows and chunks outside the panel are clipped by the
        // tensor map).
        const float dsub = p.dcoef * st.gscale;
        uint8_t* buf = tail->scratch + (size_t)(warp - 2) * STORE_BUF_BYTES;
        for (int u = u_begin; u < u_end; ++u) {
            if (lane == 0 && st.stores_in_flight > 0) {     // the previous store has finished reading `buf`
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                st.stores_in_flight = 0;
            }
            __syncwarp();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int ch = u * 2 + half;
                uint32_t v[32];
                tmem_ld32(taddr + ch * 32, v);
                tmem_ld_wait();
                const int jdc = (jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
                float gv[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float e = ex2_approx(fmaf(__uint_as_float(v[c]), p.k2, -p.k2));
                    gv[c] = fmaf(e, inv_r + tail->icol[ch * 32 + c], (c == jdc) ? -dsub : 0.f);
                }
                if (!full_tile) {     // columns past the panel edge share a stored chunk with valid ones: zero them
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (n0 + ch * 32 + c >= p.n) gv[c] = 0.f;
                }
#pragma unroll
                for (int pc = 0; pc < 4; ++pc) {         // 16-byte piece index within the 128-byte row
                    uint4 pk;
                    pk.x = pack_bf16x2(gv[pc * 8 + 0], gv[pc * 8 + 1]);
                    pk.y = pack_bf16x2(gv[pc * 8 + 2], gv[pc * 8 + 3]);
                    pk.z = pack_bf16x2(gv[pc * 8 + 4], gv[pc * 8 + 5]);
                    pk.w = pack_bf16x2(gv[pc * 8 + 6], gv[pc * 8 + 7]);
                    const int piece = half * 4 + pc;
                    *reinterpret_cast<uint4*>(buf + lane * 128 + ((piece ^ (lane & 7)) << 4)) = pk;
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(tmap_c, smem_u32(buf), 0, m0 + q * 32, (n0 >> 6) + u);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                st.stores_in_flight = 1;
            }
        }
        tc_fence_before();
        release();
    } else {   // EPI_OUT
        for (int ch = u_begin; ch < u_end; ++ch) {
            uint32_t v[32];
            tmem_ld32(taddr + ch * 32, v);
            tmem_ld_wait();
            if (rvalid) {
                const int col0 = n0 + ch * 32;
                if (p.acc_in != nullptr) {
                    const float* ap = p.acc_in + (long long)grow * p.ld_acc + col0;
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        if (col0 + c < p.n) {
                            const float4 a = *reinterpret_cast<const float4*>(ap + c);
                            v[c] = __float_as_uint(__uint_as_float(v[c]) + a.x);
                            v[c + 1] = __float_as_uint(__uint_as_float(v[c + 1]) + a.y);
                            v[c + 2] = __float_as_uint(__uint_as_float(v[c + 2]) + a.z);
                            v[c + 3] = __float_as_uint(__uint_as_float(v[c + 3]) + a.w);
                        }
                    }
                }
                if (p.out_bf16) {
                    __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)grow * p.ld_out + col0;
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        if (col0 + c < p.n) {
                            uint4 pk;
                            pk.x = pack_bf16x2(__uint_as_float(v[c]), __uint_as_float(v[c + 1]));
                            pk.y = pack_bf16x2(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
                            pk.z = pack_bf16x2(__uint_as_float(v[c + 4]), __uint_as_float(v[c + 5]));
                            pk.w = pack_bf16x2(__uint_as_float(v[c + 6]), __uint_as_float(v[c + 7]));
                            *reinterpret_cast<uint4*>(op + c) = pk;
                        }
                    }
                } else {
                    float* op = reinterpret_cast<float*>(p.out) + (long long)grow * p.ld_out + col0;
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        if (col0 + c < p.n) {
                            float4 o;
                            o.x = __uint_as_float(v[c]);
                            o.y = __uint_as_float(v[c + 1]);
                            o.z = __uint_as_float(v[c + 2]);
                            o.w = __uint_as_float(v[c + 3]);
                            *reinterpret_cast<float4*>(op + c) = o;
                        }
                    }
                }
            }
        }
        tc_fence_before();
        release();
    }
}

// Called once per epilogue thread before the CTA ends: panel stores must have been written.
template <int EPI>
__device__ __forceinline__ void epilogue_drain(const EpiState& st, int lane) {
    if (EPI == EPI_COEF && lane == 0 && st.stores_in_flight > 0) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

}  // namespace meclip
