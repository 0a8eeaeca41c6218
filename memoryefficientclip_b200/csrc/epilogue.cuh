// The three epilogues of the tile kernels, shared by the single-CTA and the CTA-pair kernel.
// Eight warps (two per TMEM lane quadrant) work on one 128-row accumulator: warp quadrant
// q = warp % 4 owns rows 32q..32q+31, warp group wg = 0/1 owns the first / second half of the
// tile's columns.  One thread = one row (tcgen05.ld 32x32b), 32 columns per load.
#pragma once
#include "sm100_ptx.cuh"

namespace meclip {

// Value summed by the forward pass: exp2(u) for the softmax losses, softplus(a)/ln2 for the sigmoid
// loss (u = a log2(e); the loss kernel multiplies by ln2 once).
// flip: the sigmoid loss takes softplus(-a) on the diagonal (the positive pair).  It is summed in
// that form, not as softplus(a) - a, so that the many tiny off-diagonal terms of a row are never
// added to a large number.
template <bool SIG>
__device__ __forceinline__ float fwd_value(float s, float fmul, float fadd, bool flip = false) {
    float u = fmaf(s, fmul, fadd);
    if (!SIG) return ex2_approx(u);
    if (flip) u = -u;
    // log2(1 + x), x = 2^-|u| in (0, 1]: lg2.approx has an ABSOLUTE error near 1, which would dominate the
    // many tiny terms of far-apart pairs, so small x uses the series x log2(e) (1 - x/2) instead
    const float x = ex2_approx(-fabsf(u));
    const float small = x * fmaf(x, -0.72134752f, 1.44269504f);
    const float big = lg2_approx(1.f + x);
    return fmaxf(u, 0.f) + (x < 0.00390625f ? small : big);
}
// Factor of the gradient coefficient: exp2(u), or sigmoid(a) = 1 / (1 + 2^-u) with u = a log2(e)
// (relative accuracy also for the very small sigmoids of far-apart pairs).
template <bool SIG>
__device__ __forceinline__ float coef_value(float s, float fmul, float fadd) {
    const float u = fmaf(s, fmul, fadd);
    if (!SIG) return ex2_approx(u);
    return rcp_approx(1.f + ex2_approx(-u));
}

template <bool SIG>
__device__ __forceinline__ void sums_chunk(const uint32_t (&v)[32], const GemmParams& p, float fmul, float fadd,
                                           bool full_tile, bool rvalid, int col_base, bool want_cols,
                                           float (&cacc)[32], float& ra0, float& ra1, float& ra2, float& ra3, int jdc) {
    if (SIG && jdc >= -1 && __any_sync(0xffffffffu, jdc >= 0)) {      // a chunk the diagonal runs through
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float e = fwd_value<SIG>(__uint_as_float(v[c]), fmul, fadd, c == jdc);
            if (!rvalid || col_base + c >= p.n) e = 0.f;
            ra0 += e;
        }
        return;
    }
    if (full_tile) {
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float e0 = fwd_value<SIG>(__uint_as_float(v[c]), fmul, fadd);
            const float e1 = fwd_value<SIG>(__uint_as_float(v[c + 1]), fmul, fadd);
            const float e2 = fwd_value<SIG>(__uint_as_float(v[c + 2]), fmul, fadd);
            const float e3 = fwd_value<SIG>(__uint_as_float(v[c + 3]), fmul, fadd);
            ra0 += e0; ra1 += e1; ra2 += e2; ra3 += e3;
            if (want_cols) { cacc[c] += e0; cacc[c + 1] += e1; cacc[c + 2] += e2; cacc[c + 3] += e3; }
        }
    } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float e = fwd_value<SIG>(__uint_as_float(v[c]), fmul, fadd);
            if (!rvalid || col_base + c >= p.n) e = 0.f;
            ra0 += e;
            if (want_cols) cacc[c] += e;
        }
    }
}

template <bool SIG>
__device__ __forceinline__ void coef_chunk(const uint32_t (&v)[32], float fmul, float fadd, float inv_r,
                                           const float* icol_chunk, float (&gv)[32]) {
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
        const float4 ic = *reinterpret_cast<const float4*>(icol_chunk + c);   // broadcast read
        gv[c] = coef_value<SIG>(__uint_as_float(v[c]), fmul, fadd) * (inv_r + ic.x);
        gv[c + 1] = coef_value<SIG>(__uint_as_float(v[c + 1]), fmul, fadd) * (inv_r + ic.y);
        gv[c + 2] = coef_value<SIG>(__uint_as_float(v[c + 2]), fmul, fadd) * (inv_r + ic.z);
        gv[c + 3] = coef_value<SIG>(__uint_as_float(v[c + 3]), fmul, fadd) * (inv_r + ic.w);
    }
}

static constexpr int COL_SLOTS = MECLIP_STRIPS ? MAX_BN / 64 : 1;   // 32-column chunks one warp group owns at most (half the tile)

struct EpiState {        // per-thread state that lives across tiles
    int stores_in_flight = 0;   // COEF: lane 0's outstanding TMA-store groups
    float gscale = 1.f;         // COEF: *grad_out (times a power of the device-resident temperature, if any)
    float fmul = 0.f, fadd = 0.f;   // the elementwise function's affine part, from the host or from device scalars
    // SUMS: column sums of this thread's row, kept in registers over a strip of tiles that share
    // their columns; reduced across rows (shuffles, shared memory, atomics) once per strip
    float cacc[COL_SLOTS][32] = {};
    int strip_n0 = -1;          // first column of the tiles accumulated so far, -1 = nothing pending
    int strip_m0 = 0;           // first row of the last tile accumulated (the slot of a deterministic flush)
};

// Per-thread set-up of the epilogue state: the affine part of the elementwise function and the
// coefficient scale, from the host values or from scalars that live on the device.
template <int EPI>
__device__ __forceinline__ void epilogue_init(const GemmParams& p, EpiState& st) {
    st.fmul = p.fmul;
    st.fadd = p.fadd;
    float gfac = 1.f;
    if (p.t_dev != nullptr) {
        const float t = __ldg(p.t_dev);
        if (p.sigmoid) {
            st.fmul = t * 1.4426950408889634f;
            if (p.b_dev != nullptr) st.fadd = __ldg(p.b_dev) * 1.4426950408889634f;
        } else {
            st.fmul = 1.4426950408889634f / t;
            st.fadd = -st.fmul;
        }
        gfac = p.g_rule == 1 ? 1.f / t : p.g_rule == 2 ? rsqrtf(t) : p.g_rule == 3 ? t : 1.f;
    }
    if (EPI == EPI_COEF) st.gscale = (p.grad_out ? __ldg(p.grad_out) : 1.f) * gfac;
}

// SUMS: add the pending column accumulators of all eight warps into col_sum and clear them.
// Every epilogue thread must call this at the same point (it uses the epilogue named barrier).
__device__ __forceinline__ void flush_column_sums(const GemmParams& p, SharedTail* tail, EpiState& st, int warp, int lane) {
    if (!MECLIP_STRIPS || st.strip_n0 < 0) return;
    const int q = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int et = (int)threadIdx.x - 64;
    const int units = p.bn >> 5;
    const int u_split = (units + 1) >> 1;
    const int u_begin = wg == 0 ? 0 : u_split;
    const int u_end = wg == 0 ? u_split : units;
    float (*colpart)[MAX_BN] = reinterpret_cast<float (*)[MAX_BN]>(tail->scratch + sizeof(tail->scratch) - 4 * MAX_BN * 4);
#pragma unroll
    for (int k = 0; k < COL_SLOTS; ++k) {
        if (u_begin + k < u_end) {
            const float cs = warp_transpose_reduce32(st.cacc[k], lane);
            colpart[q][(u_begin + k) * 32 + lane] = cs;
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) st.cacc[k][c] = 0.f;
    }
    named_bar_sync(1, EPI_THREADS);
    for (int j = et; j < p.bn; j += EPI_THREADS)
        if (st.strip_n0 + j < p.n) {
            const float v = (colpart[0][j] + colpart[1][j]) + (colpart[2][j] + colpart[3][j]);
            if (p.col_part != nullptr) p.col_part[(long long)(st.strip_m0 >> 7) * p.part_ld_cols + st.strip_n0 + j] = v;
            else atomicAdd(p.col_sum + st.strip_n0 + j, v);
        }
    named_bar_sync(1, EPI_THREADS);
    st.strip_n0 = -1;
}

// `release()` is called by every thread once its last tcgen05.ld of the tile has completed; it must
// tell the MMA issuer that this thread is done with the accumulator.
template <int EPI, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const OutDesc od, const CUtensorMap* tmap_c,
                                              SharedTail* tail, EpiState& st, uint32_t taddr, int m0, int n0,
                                              int tile_bn, int warp, int lane, Release release) {
    const int q = warp & 3;
    const int wg = EPI_WARPS == 8 ? (warp - 2) >> 2 : 0;
    const int et = (int)threadIdx.x - 64;                 // index within the epilogue group
    const int grow = m0 + q * 32 + lane;
    const bool rvalid = grow < od.m;          // od.m == p.m except for the second problem of a dual launch
    const bool full_tile = (m0 + BM <= od.m) && (n0 + p.bn <= p.n);
    // column (tile-local) on which this row meets the diagonal, -1 if outside the tile
    const long long jd_ll = (long long)grow + p.diag_shift - n0;
    const int jd = (jd_ll >= 0 && jd_ll < p.bn && n0 + jd_ll < p.n && rvalid) ? (int)jd_ll : -1;
    // this warp group's share of the columns, in units of 32 (SUMS, OUT) or 64 (COEF) columns
    // tile_bn differs from p.bn only for the narrower last column tile of a contraction (EPI_OUT)
    const int units = (EPI == EPI_COEF) ? (p.bn >> 6) : (EPI == EPI_OUT ? (tile_bn >> 5) : (p.bn >> 5));
    const int u_split = EPI_WARPS == 8 ? (units + 1) >> 1 : units;
    const int u_begin = wg == 0 ? 0 : u_split;
    const int u_end = wg == 0 ? u_split : units;

    if (EPI == EPI_SUMS && !MECLIP_STRIPS) {
        // per-tile reduction of the column sums: butterfly per 32x32 block, combine the quadrants in shared memory
        float (*colpart)[MAX_BN] = reinterpret_cast<float (*)[MAX_BN]>(tail->scratch + sizeof(tail->scratch) - 4 * MAX_BN * 4);
        const bool want_cols = p.col_sum != nullptr;
        float ra0 = 0.f, ra1 = 0.f, ra2 = 0.f, ra3 = 0.f;
        float sdiag = 0.f;
        const bool diag_here = __any_sync(0xffffffffu, jd >= 0);
        for (int ch = u_begin; ch < u_end; ++ch) {
            uint32_t v[32];
            tmem_ld32(taddr + ch * 32, v);
            tmem_ld_wait();
            if (diag_here) {
                const int jdc = (jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
#pragma unroll
                for (int c = 0; c < 32; ++c) sdiag = (c == jdc) ? __uint_as_float(v[c]) : sdiag;
            }
            float e[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) e[c] = 0.f;
            const int jdc_s = (diag_here && jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
            if (p.sigmoid) sums_chunk<true>(v, p, st.fmul, st.fadd, full_tile, rvalid, n0 + ch * 32, want_cols, e, ra0, ra1, ra2, ra3, jdc_s);
            else           sums_chunk<false>(v, p, st.fmul, st.fadd, full_tile, rvalid, n0 + ch * 32, want_cols, e, ra0, ra1, ra2, ra3, -1);
            if (want_cols) {
                const float cs = warp_transpose_reduce32(e, lane);
                colpart[q][ch * 32 + lane] = cs;
            }
        }
        tc_fence_before();
        release();
        if (rvalid && u_end > u_begin) atomicAdd(p.row_sum + grow, (ra0 + ra1) + (ra2 + ra3));
        if (jd >= 0 && (jd >> 5) >= u_begin && (jd >> 5) < u_end) p.diag[grow] = sdiag;
        if (want_cols) {
            named_bar_sync(1, EPI_THREADS);
            for (int j = et; j < p.bn; j += EPI_THREADS)
                if (n0 + j < p.n)
                    atomicAdd(p.col_sum + n0 + j, (colpart[0][j] + colpart[1][j]) + (colpart[2][j] + colpart[3][j]));
            named_bar_sync(1, EPI_THREADS);
        }
    } else if (EPI == EPI_SUMS) {
        const bool want_cols = p.col_sum != nullptr;
        if (want_cols && st.strip_n0 != n0) {       // the columns change: hand in what was accumulated
            flush_column_sums(p, tail, st, warp, lane);
            st.strip_n0 = n0;
        }
        st.strip_m0 = m0;
        float ra0 = 0.f, ra1 = 0.f, ra2 = 0.f, ra3 = 0.f;
        float sdiag = 0.f;
        const bool diag_here = __any_sync(0xffffffffu, jd >= 0);   // warp-uniform: most tiles miss the diagonal
#pragma unroll
        for (int k = 0; k < COL_SLOTS; ++k) {
            const int ch = u_begin + k;
            if (ch < u_end) {
                uint32_t v[32];
                tmem_ld32(taddr + ch * 32, v);
                tmem_ld_wait();
                if (diag_here) {
                    const int jdc = (jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
#pragma unroll
                    for (int c = 0; c < 32; ++c) sdiag = (c == jdc) ? __uint_as_float(v[c]) : sdiag;
                }
                const int jdc_s = (diag_here && jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
                if (p.sigmoid) sums_chunk<true>(v, p, st.fmul, st.fadd, full_tile, rvalid, n0 + ch * 32, want_cols, st.cacc[k], ra0, ra1, ra2, ra3, jdc_s);
                else           sums_chunk<false>(v, p, st.fmul, st.fadd, full_tile, rvalid, n0 + ch * 32, want_cols, st.cacc[k], ra0, ra1, ra2, ra3, -1);
            }
        }
        tc_fence_before();
        release();
        if (rvalid && u_end > u_begin) {
            const float rs = (ra0 + ra1) + (ra2 + ra3);
            if (p.row_part != nullptr) p.row_part[(long long)(2 * (n0 / p.bn) + wg) * p.part_ld_rows + grow] = rs;
            else atomicAdd(p.row_sum + grow, rs);
        }
        if (jd >= 0 && (jd >> 5) >= u_begin && (jd >> 5) < u_end) p.diag[grow] = sdiag;
        // deterministic mode: one slot per tile, so the column partials are handed in after every tile
        if (want_cols && p.col_part != nullptr) flush_column_sums(p, tail, st, warp, lane);
    } else if (EPI == EPI_COEF) {
        // g / c_j for the tile's columns, staged once per tile for all eight warps
        named_bar_sync(1, EPI_THREADS);            // previous tile's readers of icol are done
        for (int j = et; j < p.bn; j += EPI_THREADS) {
            float v = 0.f;
            if (p.c != nullptr && n0 + j < p.n) v = p.coef * st.gscale / __ldg(p.c + n0 + j);
            tail->icol[j] = v;
        }
        // row factor: g / r_i for the softmax losses, plain g when there are no row sums (sigmoid loss)
        const float inv_r = !rvalid ? 0.f : (p.r != nullptr ? p.coef * st.gscale / __ldg(p.r + grow) : p.coef * st.gscale);
        named_bar_sync(1, EPI_THREADS);
        // Each warp turns 32 rows x 64 columns into a 128-byte-swizzled shared tile and one lane
        // TMA-stores it (full 128-byte lines; rows and chunks outside the panel are clipped by the
        // tensor map).
        const float dsub = p.dcoef * st.gscale;
        const bool diag_here = __any_sync(0xffffffffu, jd >= 0);
        const bool want_sg = p.sg_acc != nullptr;      // sum of G_ij * S_ij for the temperature gradient
        float sg = 0.f, sg1 = 0.f;
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
                float gv[32];
                if (p.sigmoid) coef_chunk<true>(v, st.fmul, st.fadd, inv_r, &tail->icol[ch * 32], gv);
                else           coef_chunk<false>(v, st.fmul, st.fadd, inv_r, &tail->icol[ch * 32], gv);
                if (diag_here) {      // warp-uniform: only tiles that cross the diagonal pay for the correction
                    const int jdc = (jd >= 0 && (jd >> 5) == ch) ? (jd & 31) : -1;
                    if (p.sigmoid) {
                        // sigmoid(a) - 1 = -1 / (1 + 2^u), computed in that form: no cancellation for a confident pair
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const float u = fmaf(__uint_as_float(v[c]), st.fmul, st.fadd);
                            gv[c] = (c == jdc) ? -dsub * rcp_approx(1.f + ex2_approx(u)) : gv[c];
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) gv[c] -= (c == jdc) ? dsub : 0.f;
                    }
                }
                if (!full_tile) {     // columns past the panel edge share a stored chunk with valid ones: zero them
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (n0 + ch * 32 + c >= p.n) gv[c] = 0.f;
                }
                if (want_sg && rvalid) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) { sg = fmaf(gv[c], __uint_as_float(v[c]), sg); sg1 += gv[c]; }
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
        if (want_sg) {
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                sg += __shfl_xor_sync(0xffffffffu, sg, o);
                sg1 += __shfl_xor_sync(0xffffffffu, sg1, o);
            }
            if (lane == 0) { atomicAdd(p.sg_acc, sg); atomicAdd(p.sg_acc + 1, sg1); }
        }
    } else {   // EPI_OUT
        // Wide tiles (two MMAs per K step, see GemmParams::wide): the first MMA's 256 accumulator columns hold the
        // first 128 B rows of CTA 0 and of CTA 1, the second MMA's columns (from TMEM column 256) the remaining rows
        // of each, so accumulator chunk ch maps to tile columns through the four pieces below.  For tiles of up
        // to 256 columns the map is the identity.
        const int n1 = tile_bn < MAX_BN ? tile_bn : MAX_BN, n2 = tile_bn - n1, h1 = n1 >> 1, half = tile_bn >> 1;
        for (int ch = u_begin; ch < u_end; ++ch) {
            const int c = ch * 32;
            int tcol = c, gcol = c;
            if (p.wide && tile_bn > MAX_BN) {
                if (c < n1) {
                    gcol = c < h1 ? c : half + (c - h1);
                } else {
                    const int c2 = c - n1;
                    tcol = MAX_BN + c2;
                    gcol = c2 < (n2 >> 1) ? h1 + c2 : half + h1 + (c2 - (n2 >> 1));
                }
            }
            uint32_t v[32];
            tmem_ld32(taddr + tcol, v);
            tmem_ld_wait();
            if (rvalid) {
                const int col0 = n0 + gcol;
                if (od.acc_in != nullptr) {
                    const float* ap = od.acc_in + (long long)grow * od.ld_acc + col0;
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
                if (od.out_bf16) {
                    __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(od.out) + (long long)grow * od.ld_out + col0;
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
                    float* op = reinterpret_cast<float*>(od.out) + (long long)grow * od.ld_out + col0;
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
// (Pending column sums are flushed by the kernels, which know whether the tile loop ended cleanly.)
template <int EPI>
__device__ __forceinline__ void epilogue_drain(const EpiState& st, int lane) {
    if (EPI == EPI_COEF && lane == 0 && st.stores_in_flight > 0) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

}  // namespace meclip
