// libmeclip_sm100.so: host launchers and the C ABI declared in include/meclip.h.
// Device code: umma_gemm.cuh (tcgen05 tile kernels) and the row kernels below.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>
#include <string>

#include <nvtx3/nvToolsExt.h>

#include "../../include/meclip.h"
#include "umma_gemm.cuh"
#include "umma_gemm2.cuh"

namespace meclip {

// ------------------------------------------------------------------------------------
// error bookkeeping
// ------------------------------------------------------------------------------------
static std::mutex g_err_mutex;
static std::string g_last_error;

static int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    std::lock_guard<std::mutex> lock(g_err_mutex);
    g_last_error = buf;
    return code;
}

#define MECLIP_CUDA(expr)                                                                         \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess) {                                                                 \
            cudaGetLastError(); /* reported here: do not leave it for the next launch's check */  \
            return fail(MECLIP_ECUDA, "%s: %s", #expr, cudaGetErrorString(e__));                  \
        }                                                                                         \
    } while (0)

// ------------------------------------------------------------------------------------
// launch counter and optional per-kernel CUDA-event timing
// ------------------------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
// tags >= TAG_ROW are HBM-bound passes: their `flops` field carries algorithmic BYTES (read + written)
enum { TAG_SUMS = 0, TAG_COEF = 1, TAG_DX = 2, TAG_DY = 3, TAG_ROW = 4, TAG_NORM_FWD = 5, TAG_NORM_BWD = 6,
       TAG_TRANSPOSE = 7, TAG_ACCUM = 8, TAG_COUNT = 9 };
struct ProfileRecord { int tag; cudaEvent_t start, stop; double flops; };
static std::mutex g_prof_mutex;
static bool g_prof_on = false;
static std::vector<ProfileRecord> g_prof;
static thread_local int t_tag = TAG_ROW;

struct ScopedTiming {   // brackets one launch with events on its stream while profiling is on
    cudaStream_t s; bool on; ProfileRecord rec;
    ScopedTiming(cudaStream_t stream, int tag, double flops) : s(stream), on(false) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        std::lock_guard<std::mutex> lock(g_prof_mutex);
        if (!g_prof_on) return;
        rec.tag = tag; rec.flops = flops;
        if (cudaEventCreate(&rec.start) != cudaSuccess) return;
        if (cudaEventCreate(&rec.stop) != cudaSuccess) { cudaEventDestroy(rec.start); return; }
        cudaEventRecord(rec.start, s);
        on = true;
    }
    ~ScopedTiming() {
        if (!on) return;
        cudaEventRecord(rec.stop, s);
        std::lock_guard<std::mutex> lock(g_prof_mutex);
        g_prof.push_back(rec);
    }
};

// NVTX range around an entry point (header-only NVTX: a no-op unless a profiler is attached)
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};

// test hook: device buffer for the in-kernel trace of CTA 0 (null = off)
static unsigned long long* g_trace_buf = nullptr;
static unsigned int g_trace_capacity = 0;

// Scalars that live on the device (learnable temperature, logit scale / bias): bound by
// meclip_bind_device_scalars for the next tile-pass call of the same host thread, consumed by it.
struct DeviceScalars { const float* t = nullptr; const float* b = nullptr; int g_rule = 0; };
static thread_local DeviceScalars t_scalars;
static DeviceScalars take_scalars() {
    const DeviceScalars ds = t_scalars;
    t_scalars = DeviceScalars();
    return ds;
}

// Bound of every barrier wait inside the tile kernels: 2 s unless MECLIP_WAIT_LIMIT_MS says otherwise
// (a context that is time-sliced with other processes for longer than the limit would trip it spuriously).
static unsigned long long wait_limit_ns() {
    static const unsigned long long ns = []() -> unsigned long long {
        const char* v = std::getenv("MECLIP_WAIT_LIMIT_MS");
        const long long ms = v ? std::atoll(v) : 0;
        return ms > 0 ? (unsigned long long)ms * 1000000ull : WAIT_LIMIT_NS;
    }();
    return ns;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------------------------
// row kernels: one warp per row, 16-byte vector accesses (HBM-bound passes)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ float load1(const float* p) { return *p; }
__device__ __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store8(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

static constexpr int ROW_KERNEL_THREADS = 256;

// x_hat = x / max(||x||, 1e-12) as bf16 (+ inv_norm); normalize == 0: dtype conversion only.
// The output row has dpad = round_up(d, 8) columns, the ones past d are zero, so that the tile kernels
// always see 16-byte rows.  vec == 0 (d not a multiple of 8, or an unaligned input): element-wise reads.
template <typename TIn>
__device__ __forceinline__ void normalize_fwd_row(const TIn* __restrict__ x, long long ldx, long long rows, int d, int dpad,
                                                  int normalize, int vec, __nv_bfloat16* __restrict__ out, long long ldh,
                                                  float* __restrict__ inv_norm) {
    const long long row = (long long)blockIdx.x * (ROW_KERNEL_THREADS / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const TIn* xr = x + row * ldx;
    float inv = 1.f;
    if (normalize) {
        float ss = 0.f;
        if (vec) {
            for (int c = lane * 8; c < d; c += 256) {
                float v[8];
                load8(xr + c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
            }
        } else {
            for (int c = lane; c < d; c += 32) { const float v = load1(xr + c); ss = fmaf(v, v, ss); }
        }
        ss = warp_sum(ss);
        inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
        if (lane == 0 && inv_norm != nullptr) inv_norm[row] = inv;
    }
    __nv_bfloat16* orow = out + row * ldh;
    if (vec) {
        for (int c = lane * 8; c < d; c += 256) {
            float v[8];
            load8(xr + c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= inv;
            store8(orow + c, v);
        }
    } else {
        for (int c = lane; c < dpad; c += 32) store1(orow + c, c < d ? load1(xr + c) * inv : 0.f);
    }
}

template <typename TIn>
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
normalize_fwd_kernel(const TIn* __restrict__ x, long long ldx, long long rows, int d, int dpad, int normalize, int vec,
                     __nv_bfloat16* __restrict__ out, long long ldh, float* __restrict__ inv_norm) {
    normalize_fwd_row<TIn>(x, ldx, rows, d, dpad, normalize, vec, out, ldh, inv_norm);
}

// Both inputs of a step in one launch (blockIdx.y = 0: first matrix, 1: second matrix; same shape and dtype).
template <typename TIn>
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
normalize_fwd_pair_kernel(const TIn* __restrict__ x0, long long ld0, int vec0, __nv_bfloat16* __restrict__ out0,
                          float* __restrict__ inv0, const TIn* __restrict__ x1, long long ld1, int vec1,
                          __nv_bfloat16* __restrict__ out1, float* __restrict__ inv1, long long rows, int d, int dpad,
                          int normalize, long long ldh) {
    if (blockIdx.y == 0) normalize_fwd_row<TIn>(x0, ld0, rows, d, dpad, normalize, vec0, out0, ldh, inv0);
    else                 normalize_fwd_row<TIn>(x1, ld1, rows, d, dpad, normalize, vec1, out1, ldh, inv1);
}

// dx = (g - x_hat (x_hat . g)) * inv_norm; inv_norm == nullptr: dx = g (dtype conversion of a gradient).
// g and x_hat are this library's own 16-byte-aligned buffers; vec_out == 0: element-wise stores of dx.
template <typename TG, typename TOut>
__device__ __forceinline__ void normalize_bwd_row(const TG* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ xh,
                                                  long long ldh, const float* __restrict__ inv_norm, long long rows, int d,
                                                  int vec_out, TOut* __restrict__ dx, long long lddx) {
    const long long row = (long long)blockIdx.x * (ROW_KERNEL_THREADS / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const TG* gr = g + row * ldg;
    const __nv_bfloat16* hr = xh + row * ldh;
    const bool jac = inv_norm != nullptr;
    float dot = 0.f;
    if (jac) {
        const int dpad = (d + 7) & ~7;          // x_hat is zero past d, so the padded columns add nothing
        for (int c = lane * 8; c < dpad; c += 256) {
            float gv[8], hv[8];
            load8(gr + c, gv);
            load8(hr + c, hv);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(gv[i], hv[i], dot);
        }
        dot = warp_sum(dot);
    }
    const float inv = jac ? inv_norm[row] : 1.f;
    TOut* orow = dx + row * lddx;
    if (vec_out) {
        for (int c = lane * 8; c < d; c += 256) {
            float gv[8], hv[8];
            load8(gr + c, gv);
            if (jac) {
                load8(hr + c, hv);
#pragma unroll
                for (int i = 0; i < 8; ++i) gv[i] = (gv[i] - hv[i] * dot) * inv;
            }
            store8(orow + c, gv);
        }
    } else {
        for (int c = lane; c < d; c += 32) {
            float v = load1(gr + c);
            if (jac) v = (v - load1(hr + c) * dot) * inv;
            store1(orow + c, v);
        }
    }
}

template <typename TG, typename TOut>
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
normalize_bwd_kernel(const TG* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ xh, long long ldh,
                     const float* __restrict__ inv_norm, long long rows, int d, int vec_out, TOut* __restrict__ dx,
                     long long lddx) {
    normalize_bwd_row<TG, TOut>(g, ldg, xh, ldh, inv_norm, rows, d, vec_out, dx, lddx);
}

// Both gradients of a step in one launch (blockIdx.y selects); fp32 contraction outputs in, the inputs' dtype out.
template <typename TOut>
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
normalize_bwd_pair_kernel(const float* __restrict__ g0, const __nv_bfloat16* __restrict__ xh0, const float* __restrict__ inv0,
                          int vec0, TOut* __restrict__ dx0, long long lddx0, const float* __restrict__ g1,
                          const __nv_bfloat16* __restrict__ xh1, const float* __restrict__ inv1, int vec1,
                          TOut* __restrict__ dx1, long long lddx1, long long ldg, long long ldh, long long rows, int d) {
    if (blockIdx.y == 0) normalize_bwd_row<float, TOut>(g0, ldg, xh0, ldh, inv0, rows, d, vec0, dx0, lddx0);
    else                 normalize_bwd_row<float, TOut>(g1, ldg, xh1, ldh, inv1, rows, d, vec1, dx1, lddx1);
}

// ---- LiT in one tile pass (its coefficients separate: G_ij = g E_ij / r_i - g [i == j]) -----------------
// y[row][col] = 1, y[row][col+1 .. col+7] = 0: the ones column that makes the contraction E [Y | 1] also
// produce the row sums of E.
__global__ void __launch_bounds__(256)
ones_column_kernel(__nv_bfloat16* __restrict__ y, long long rows, long long col, long long ld) {
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    uint4 v = make_uint4(0x00003F80u, 0u, 0u, 0u);       // bf16 1.0 in the low half, seven zeros
    *reinterpret_cast<uint4*>(y + r * ld + col) = v;
}

// row_sum[i] = U[i][d] (the ones column), diag[i] = <x_i, y_i>: what the loss needs besides U.
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
lit_fused_stats_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ y, long long ldy,
                       const float* __restrict__ u, long long ldu, long long rows, int d, float* __restrict__ row_sum,
                       float* __restrict__ diag) {
    const long long row = (long long)blockIdx.x * (ROW_KERNEL_THREADS / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float dot = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        float a[8], b[8];
        load8(x + row * ldx + c, a);
        load8(y + row * ldy + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(a[i], b[i], dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) {
        diag[row] = dot;
        row_sum[row] = u[row * ldu + d];
    }
}

// dx[i][:] = g (U[i][:] / r_i - y[i][:]) over the first d columns, g = grad_scale * (*grad_out).
template <typename TOut>
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
lit_fused_bwd_kernel(const float* __restrict__ u, long long ldu, const __nv_bfloat16* __restrict__ y, long long ldy,
                     const float* __restrict__ row_sum, const float* __restrict__ grad_out, float grad_scale,
                     const float* __restrict__ t_dev, int g_rule, long long rows,
                     int d, int vec_out, TOut* __restrict__ dx, long long lddx) {
    const long long row = (long long)blockIdx.x * (ROW_KERNEL_THREADS / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float g = grad_scale * (grad_out != nullptr ? __ldg(grad_out) : 1.f);
    if (t_dev != nullptr) {       // temperature on the device: grad_scale was formed with T = 1
        const float t = __ldg(t_dev);
        g *= g_rule == 1 ? 1.f / t : g_rule == 2 ? rsqrtf(t) : 1.f;
    }
    const float gr = g / __ldg(row_sum + row);
    const float* ur = u + row * ldu;
    const __nv_bfloat16* yr = y + row * ldy;
    TOut* orow = dx + row * lddx;
    if (vec_out) {
        for (int c = lane * 8; c < d; c += 256) {
            float uv[8], yv[8];
            load8(ur + c, uv);
            load8(yr + c, yv);
#pragma unroll
            for (int i = 0; i < 8; ++i) uv[i] = fmaf(uv[i], gr, -g * yv[i]);
            store8(orow + c, uv);
        }
    } else {
        for (int c = lane; c < d; c += 32) store1(orow + c, fmaf(ur[c], gr, -g * load1(yr + c)));
    }
}

// out[c][r] = in[r][c] for a bf16 matrix: 64 x 64 tiles through shared memory, 16-byte global accesses.
// The contractions read X^T / Y^T as K-major B operands (K-major tiles feed the tensor cores
// measurably faster than MN-major ones when A is the transposed panel).
// One CTA moves a 64 x 64 tile with 16-byte global accesses on both sides.  Shared memory holds the tile
// already transposed as 32-bit words T[c][p] = (in[2p][c], in[2p+1][c]); the word index is XOR-swizzled by the
// 8-column chunk of c in units of four words, which makes the 32-bit stores of a warp (8 chunks x 4 row pairs)
// and the 16-byte loads of the write-out hit all 32 banks once.
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, long long rows, int cols,
                      __nv_bfloat16* __restrict__ out, long long ld_out) {
    __shared__ __align__(16) uint32_t tile[64][32];
    const long long r0 = (long long)blockIdx.x * 64;
    const int c0 = blockIdx.y * 64;
    const int t = threadIdx.x;
    {
        const int k = t & 7;                  // 8-column chunk of the input row
        const int rp = t >> 3;                // row pair
        const long long r = r0 + 2 * rp;
        const int c = c0 + 8 * k;
        uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
        if (c < cols) {                       // cols is a multiple of 8: a chunk is inside or outside as a whole
            if (r < rows) a = __ldg(reinterpret_cast<const uint4*>(in + r * ld_in + c));
            if (r + 1 < rows) b = __ldg(reinterpret_cast<const uint4*>(in + (r + 1) * ld_in + c));
        }
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        const int pw = rp ^ (k << 2);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            tile[8 * k + 2 * m][pw] = __byte_perm(aw[m], bw[m], 0x5410);
            tile[8 * k + 2 * m + 1][pw] = __byte_perm(aw[m], bw[m], 0x7632);
        }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int oc = (t >> 3) + h * 32;     // output row = input column
        const int g = t & 7;                  // 8 consecutive output columns = input rows 8g .. 8g+7
        // rows is padded to a multiple of 8 in ld_out, so a 16-byte store stays inside the pitch
        if (c0 + oc < cols && r0 + 8 * g < rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(&tile[oc][4 * (g ^ ((oc >> 3) & 7))]);
            *reinterpret_cast<uint4*>(out + (long long)(c0 + oc) * ld_out + r0 + 8 * g) = v;
        }
    }
}

// dst[i] += src[i], fp32, 16-byte accesses (the owner of a text shard adds the partial
// gradient another rank of the ring sent it).
__global__ void __launch_bounds__(256)
accumulate_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n4) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 a = reinterpret_cast<float4*>(dst)[i];
        const float4 b = reinterpret_cast<const float4*>(src)[i];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        reinterpret_cast<float4*>(dst)[i] = a;
    }
}

// dst[i] += src_0[i] + src_1[i] + ... (added in that order), the sources `stride4` float4 apart: the owner of a
// text shard adds the world-1 partial gradients of one backward in one pass over its gradient.
__global__ void __launch_bounds__(256)
accumulate_many_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, int n_src, long long stride4,
                           long long n4) {
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += step) {
        float4 a = reinterpret_cast<float4*>(dst)[i];
        for (int s = 0; s < n_src; ++s) {
            const float4 b = reinterpret_cast<const float4*>(src)[(long long)s * stride4 + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        reinterpret_cast<float4*>(dst)[i] = a;
    }
}

// out[i] += parts[0][i] + parts[1][i] + ... in that order (deterministic forward: the slots of the partial sums).
__global__ void __launch_bounds__(256)
reduce_parts_kernel(const float* __restrict__ parts, int n_slots, long long ld, long long n, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int k = 0; k < n_slots; ++k) acc += parts[(long long)k * ld + i];
    out[i] += acc;
}

// loss (+)= scale * sum_i [ w (log r_i + log c_i) - (s_ii - 1)/T ]: one block, fixed order.
__global__ void __launch_bounds__(1024)
loss_finalize_kernel(const float* __restrict__ r, const float* __restrict__ c, const float* __restrict__ diag,
                     long long n, float inv_t, const float* __restrict__ t_dev, float scale, int accumulate,
                     float* __restrict__ loss) {
    __shared__ double part[1024];
    double acc = 0.0;
    if (t_dev != nullptr) inv_t = 1.f / __ldg(t_dev);       // a temperature that lives on the device
    // eight independent elements per thread and trip, so that the loads of a trip are all in flight together
    // (one block with one load at a time is bound by the load latency); out-of-range slots contribute 0
    for (long long i0 = threadIdx.x; i0 < n; i0 += 8 * 1024) {
        float rv[8], cv[8], dv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const long long i = i0 + (long long)u * 1024;
            const bool in = i < n;
            rv[u] = in ? __ldg(r + i) : 1.f;
            cv[u] = (in && c != nullptr) ? __ldg(c + i) : 1.f;
            dv[u] = in ? __ldg(diag + i) : 1.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            // lg2.approx (absolute error 2^-22, the sums themselves come from ex2.approx) instead of logf: the
            // single block is instruction-bound and logf costs about 30 instructions; fp64 accumulation
            float t = lg2_approx(rv[u]);
            if (c != nullptr) t = 0.5f * (t + lg2_approx(cv[u]));
            acc += (double)(0.6931471805599453f * t) - (double)((dv[u] - 1.f) * inv_t);
        }
    }
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if ((int)threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float v = (float)(part[0] * (double)scale);
        *loss = accumulate ? *loss + v : v;
    }
}

// Sigmoid loss: loss (+)= scale * ln2 * sum_i row_sum_i, where row_sum_i holds
// [ sum_{j != i} softplus(a_ij) + softplus(-a_ii) ] / ln2 (the tile pass flips the diagonal's sign).
__global__ void __launch_bounds__(1024)
siglip_finalize_kernel(const float* __restrict__ r, const float* __restrict__ diag, long long n, float t, float b,
                       float scale, int accumulate, float* __restrict__ loss) {
    __shared__ double part[1024];
    double acc = 0.0;
    for (long long i0 = threadIdx.x; i0 < n; i0 += 8 * 1024) {
        float rv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const long long i = i0 + (long long)u * 1024;
            rv[u] = i < n ? __ldg(r + i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += 0.6931471805599453 * (double)rv[u];
    }
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if ((int)threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float v = (float)(part[0] * (double)scale);
        *loss = accumulate ? *loss + v : v;
    }
}

// Test hook: a bounded wait that is meant to run out.  One CTA initialises an mbarrier nobody ever arrives
// on and waits on it with the tile kernels' own wait routine; when the limit has passed the wait returns
// false, the CTA records that in the status word and ends normally (no TMA, no tensor memory involved).
__global__ void __launch_bounds__(64)
wait_probe_kernel(unsigned long long limit_ns, int* __restrict__ status) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
    }
    __syncthreads();
    // warp 0 waits on its own time limit, warp 1 also watches the abort flag (the two ways a role gives up)
    const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, threadIdx.x >= 32, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_flag) && status != nullptr) atomicExch(status, 1);
}

// ------------------------------------------------------------------------------------
// TMA descriptors
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// bf16 matrix, row-major: `outer` rows of `inner` contiguous elements, pitch ld elements.
// Box = box_inner (64 elements = 128 bytes, swizzled) x box_outer rows.
// f32: the elements are fp32 (box_inner then counts 4-byte elements: 32 of them are the 128 swizzled bytes).
static int make_tmap(CUtensorMap* tm, const void* base, long long inner, long long outer, long long ld, int box_inner,
                     int box_outer, bool f32 = false) {
    EncodeTiledFn enc = get_encode_fn();
    if (enc == nullptr) return fail(MECLIP_EUNSUPPORTED, "cuTensorMapEncodeTiled not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MECLIP_ECUDA, "cuTensorMapEncodeTiled failed (%d) inner=%lld outer=%lld ld=%lld box=%dx%d", (int)r,
                    inner, outer, ld, box_inner, box_outer);
    return MECLIP_OK;
}

// Coefficient panel in its column-blocked layout: chunk c (64 columns) is a contiguous
// [rows_alloc x 64] bf16 slab.  Tensor map dims {64, rows, chunks}; box {64, box_rows, 1}.
static int make_tmap_blocked(CUtensorMap* tm, const void* base, long long rows, long long chunks, long long rows_alloc,
                             int box_rows, long long chunks_alloc) {
    EncodeTiledFn enc = get_encode_fn();
    if (enc == nullptr) return fail(MECLIP_EUNSUPPORTED, "cuTensorMapEncodeTiled not available from this driver");
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)chunks};
    cuuint64_t strides[2] = {128, (cuuint64_t)rows_alloc * 128};
    (void)chunks_alloc;
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MECLIP_ECUDA, "cuTensorMapEncodeTiled (blocked panel) failed (%d) rows=%lld chunks=%lld alloc=%lld box=%d",
                    (int)r, rows, chunks, rows_alloc, box_rows);
    return MECLIP_OK;
}

static int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Also binds the runtime's primary context to the calling thread: the tensor-map encoder is a
// driver-API entry point and fails with "invalid context" on a thread that has made no runtime
// call yet (PyTorch's autograd thread on its first backward).
static int check_device() {
    static int supported[64] = {0};   // 0 unknown, 1 ok, -1 unsupported
    int dev = 0;
    MECLIP_CUDA(cudaGetDevice(&dev));
    MECLIP_CUDA(cudaSetDevice(dev));
    if (dev < 0 || dev >= 64) return fail(MECLIP_EUNSUPPORTED, "device index %d out of range", dev);
    if (supported[dev] == 0) {
        int major = 0;
        MECLIP_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        supported[dev] = (major == 10) ? 1 : -1;
    }
    if (supported[dev] < 0) return fail(MECLIP_EUNSUPPORTED, "device %d is not sm_100: these kernels are sm_100a only", dev);
    return MECLIP_OK;
}

// Tile width for an N extent: least padding first, then the wider tile.
static int pick_bn(long long n) {
    const int cand[4] = {256, 192, 128, 64};
    int best = 64;
    long long best_pad = -1;
    for (int i = 0; i < 4; ++i) {
        const long long tiles = (n + cand[i] - 1) / cand[i];
        const long long pad = tiles * cand[i] - n;
        if (best_pad < 0 || pad < best_pad) { best_pad = pad; best = cand[i]; }
    }
    return best;
}

// Column-tile width of a contraction (m rows, n columns).  Kernels that share the GPU (side streams,
// dynamic tiles) fill each other's last wave, so there the widest tile wins; a kernel that runs alone
// pays for a partly filled last wave, so there the width is chosen by waves x tile cost.
static int pair_mode();

// MECLIP_WIDE=1 runs the contractions on wide CTA-pair tiles (GemmParams::wide).  Off by default: measured at
// B = 32768, D = 1152 (3 x 384 columns instead of 4 x 256 + 128), same GPU and call: dX / dY alone 960 / 963
// against 1016 / 1018 TFLOP/s, step 8.85-8.92 against 8.87-8.88 ms.  The 17 % fewer operand bytes per FLOP do
// not pay for the accumulator that can no longer be double-buffered and the shallower operand ring (5 stages
// of 40 KiB); the kernels are kept, and unit-tested, as that measured alternative.
static bool wide_allowed() {
    static const bool on = []() { const char* v = std::getenv("MECLIP_WIDE"); return v && v[0] == '1'; }();
    return on;
}

// Width of a wide CTA-pair tile (a multiple of 64 in (256, 512], see GemmParams::wide) for n > 256 output
// columns: the width whose tiles cover n with the fewest computed columns (the last tile may be narrower, in
// steps of 32 up to 256 and of 64 beyond); wider on ties.  1152 -> 3 x 384, 1024 -> 2 x 512, 768 -> 2 x 384.
static int pick_wide_bn(long long n) {
    int best = 256;
    long long best_cost = -1;
    for (int bn = 512; bn >= 320; bn -= 64) {
        const long long tiles = (n + bn - 1) / bn;
        const long long rest = n - (tiles - 1) * bn;
        const long long last = rest > 256 ? (rest + 63) / 64 * 64 : (rest + 31) / 32 * 32;
        const long long cost = (tiles - 1) * bn + last;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

static int pick_contraction_bn(long long m, long long n, bool shares_gpu, bool b_k_major) {
    if (n < 256) return pick_bn(n);
    if (shares_gpu) return 256;
    // CTA pairs: 256-wide tiles even when alone (measured: a 192-wide pair tile loses more per column than the
    // fuller last wave gains: dX 960 vs 1127 TFLOP/s, dY 915 vs 923 at B = 32768, D = 1152)
    if (b_k_major && pair_mode() != 0) return wide_allowed() ? pick_wide_bn(n) : 256;
    // measured: a 192-wide tile costs ~7 % more per column than a 256-wide one; the narrower ones (more cost per
    // column still: less reuse of the A tile) only pay when the wide tiles would leave most SMs without work,
    // i.e. for the small problems of the whole-step path (4096 x 512 outputs: 64 tiles of 256 columns on 148 SMs)
    const int cand[4] = {256, 192, 128, 64};
    const double cost_per_col[4] = {1.0, 1.07, 1.2, 1.5};
    int best = 256;
    double best_t = 0.0;
    for (int i = 0; i < 4; ++i) {
        const long long tiles = ((m + BM - 1) / BM) * ((n + cand[i] - 1) / cand[i]);
        const long long waves = (tiles + sm_count() - 1) / sm_count();
        const double t = (double)waves * cand[i] * cost_per_col[i];
        if (i == 0 || t < best_t) { best_t = t; best = cand[i]; }
    }
    return best;
}

// ------------------------------------------------------------------------------------
// GEMM launcher
// ------------------------------------------------------------------------------------
struct Operand {
    const void* ptr;
    long long ld;      // elements
    bool mn_major;     // false: [extent rows][K contiguous]; true: [K rows][extent contiguous]
    // > 0: the operand is a coefficient panel in column-blocked layout with this many allocated rows
    // per 64-column chunk (ld then holds the allocated chunk count); only for the A operand
    long long blocked_rows_alloc = 0;
    // fp32 elements, multiplied as tf32 (K-major, sums and coefficient passes only; A and B together)
    bool f32 = false;
};

template <int EPI, bool A_MN, bool B_MN>
static int launch_gemm_t(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                         size_t smem_bytes, cudaStream_t stream) {
    auto kern = umma_gemm_kernel<EPI, A_MN, B_MN>;
    MECLIP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    const int tiles = p.num_m_tiles * p.num_n_tiles;
    const int units = (tiles + p.strip_len - 1) / p.strip_len;
    const int grid = units < sm_count() ? units : sm_count();
    ScopedTiming timing(stream, t_tag, 2.0 * p.m * p.n * p.k);
    kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(ta, tb, tc, p);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

template <int EPI, int A_MODE, bool TF32 = false>
static int launch_pair_t(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                         size_t smem_bytes, cudaStream_t stream, const CUtensorMap* td_opt = nullptr, double flops = -1.0) {
    auto kern = umma_gemm_pair_kernel<EPI, A_MODE, TF32>;
    const CUtensorMap& td = td_opt != nullptr ? *td_opt : tb;
    MECLIP_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    // how many CTA pairs the device can hold at once (an SM without a free neighbour cannot host one)
    static int max_clusters[64] = {0};
    int dev = 0;
    MECLIP_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && max_clusters[dev] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * sm_count());
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = SMEM_LIMIT;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count() / 2; }
        max_clusters[dev] = n;
    }
    const int cap = (dev >= 0 && dev < 64) ? max_clusters[dev] : sm_count() / 2;
    const int tiles = p.dual ? p.tiles0 + p.num_m_tiles2 * p.num_n_tiles : p.num_m_tiles * p.num_n_tiles;
    const int units = (tiles + p.strip_len - 1) / p.strip_len;
    const int clusters = units < cap ? units : cap;
    ScopedTiming timing(stream, t_tag, flops >= 0.0 ? flops : 2.0 * p.m * p.n * p.k);
    kern<<<2 * clusters, GEMM_THREADS, smem_bytes, stream>>>(ta, tb, tc, td, p);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

// MECLIP_PAIR: unset = auto (below), 0 = single-CTA kernels only, 1 = CTA pairs (256 x bn tiles, cta_group::2)
// wherever B is K-major, 2 = CTA pairs for the two contractions only.  A pair stages 32 KiB per CTA and K-step
// instead of 48 KiB, so six stages fit instead of four, but every tile pays a few cross-CTA round trips.
// Measured on the power-capped step at B = 32768 (ms, modes 0 / 1 / 2, same GPU and call): D = 256 2.96 / 3.14 /
// 2.81, D = 512 4.33 / 4.55 / 4.30, D = 640 5.51 / 5.59 / 5.35, D = 768 6.12 / 6.06 / 6.06, D = 1152 9.25 / 8.59 /
// 8.94.  Auto: the contractions (K = panel width, thousands) always run as pairs; the sums and coefficient
// passes (K = D) do from PAIR_MIN_K on.
static constexpr long long PAIR_MIN_K = 800;
static int pair_mode() {
    static const int mode = []() {
        const char* v = std::getenv("MECLIP_PAIR");
        if (v == nullptr || v[0] == '\0') return -1;      // auto
        return std::atoi(v);
    }();
    return mode;
}

// `panel` (EPI_COEF only): the bf16 output panel [m x n], column-blocked with panel_rows_alloc rows
// per chunk, written by TMA stores.
static int launch_gemm(int epi, const Operand& a, const Operand& b, long long m, long long n, long long k, int bn,
                       GemmParams p, cudaStream_t stream, void* panel = nullptr, long long panel_rows_alloc = 0,
                       long long panel_chunks_alloc = 0) {
    if (m < 1 || n < 1 || k < 1) return fail(MECLIP_EINVAL, "gemm extents must be >= 1 (m=%lld n=%lld k=%lld)", m, n, k);
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return fail(MECLIP_EINVAL, "gemm extent exceeds 2^31");
    const bool wide = bn > MAX_BN;      // two MMAs per K step, CTA-pair kernel, plain contraction only
    if (bn < 32 || bn > 2 * MAX_BN || bn % 32 != 0 || ((b.mn_major || epi == EPI_COEF || wide) && bn % 64 != 0) ||
        (wide && (epi != EPI_OUT || b.mn_major || g_trace_buf != nullptr || pair_mode() == 0)))
        return fail(MECLIP_EINVAL, "tile width %d not supported", bn);
    const bool f32 = a.f32;
    if (f32) {
        // fp32 operands read as tf32: the CTA-pair kernel with K-major A and B, 32 elements per K step
        if (!b.f32 || a.mn_major || b.mn_major || a.blocked_rows_alloc > 0 || epi == EPI_OUT || wide || bn % 64 != 0 ||
            g_trace_buf != nullptr)
            return fail(MECLIP_EINVAL, "fp32 operands: sums and coefficient passes with K-major A and B only");
        if (!aligned16(a.ptr) || !aligned16(b.ptr) || a.ld % 4 != 0 || b.ld % 4 != 0)
            return fail(MECLIP_EINVAL, "fp32 operands must be 16-byte aligned with pitches that are multiples of 4 elements");
    } else if (b.f32) {
        return fail(MECLIP_EINVAL, "fp32 operands: A and B together");
    } else
    if (!aligned16(a.ptr) || !aligned16(b.ptr) || (a.blocked_rows_alloc == 0 && a.ld % 8 != 0) || b.ld % 8 != 0)
        return fail(MECLIP_EINVAL, "operands must be 16-byte aligned with pitches that are multiples of 8 elements");
    const int bk = f32 ? BK / 2 : BK;         // elements per K step: 128 bytes per row either way
    CUtensorMap ta, tb, tc;
    int rc;
    if (a.blocked_rows_alloc > 0) {
        // panel of G [rows x cols]: as A = G (K-major) rows = m, cols = k; as A = G^T (MN-major) rows = k, cols = m
        if (a.mn_major) rc = make_tmap_blocked(&ta, a.ptr, k, (m + 63) / 64, a.blocked_rows_alloc, BK, a.ld);
        else            rc = make_tmap_blocked(&ta, a.ptr, m, (k + 63) / 64, a.blocked_rows_alloc, BM, a.ld);
        p.a_blocked = 1;
    } else if (a.mn_major) rc = make_tmap(&ta, a.ptr, m, k, a.ld, 64, BK);
    else                   rc = make_tmap(&ta, a.ptr, k, m, a.ld, bk, BM, f32);
    if (rc) return rc;
    // CTA pairs (256 x bn tiles) whenever B is K-major; the single-CTA kernel keeps MN-major B
    const int pmode = pair_mode();
    const bool pair = !b.mn_major && bn % 64 == 0 && g_trace_buf == nullptr &&      // the in-kernel trace is a single-CTA hook
                      (f32 || wide || pmode == 1 || ((pmode == 2 || pmode < 0) && epi == EPI_OUT && bn == 256) ||
                       (pmode < 0 && epi != EPI_OUT && bn == 256 && k >= PAIR_MIN_K));
    if (b.mn_major) rc = make_tmap(&tb, b.ptr, n, k, b.ld, 64, BK);
    else            rc = make_tmap(&tb, b.ptr, k, n, b.ld, bk, pair ? bn / 2 : bn, f32);
    if (rc) return rc;
    if (epi == EPI_COEF) {
        if (panel == nullptr || !aligned16(panel) || panel_rows_alloc < m) return fail(MECLIP_EINVAL, "coefficient panel misaligned");
        rc = make_tmap_blocked(&tc, panel, m, (n + 63) / 64, panel_rows_alloc, 32, panel_chunks_alloc);   // one warp's 32 rows x 64 columns per store
        if (rc) return rc;
    } else {
        tc = ta;
    }
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.bn = bn;
    p.num_m_tiles = (int)((m + BM - 1) / BM);
    p.num_n_tiles = (int)((n + bn - 1) / bn);
    p.k_steps = (int)((k + bk - 1) / bk);
    p.trace = g_trace_buf;
    p.trace_capacity = g_trace_capacity;
    p.wait_limit_ns = wait_limit_ns();
    // Tile ids walk group_m row tiles of one column tile, then the next column tile.  The sums pass wants tall
    // groups (a strip shares its columns).  A contraction streams its A operand (the coefficient panel) from HBM:
    // with short groups the column tiles that share panel rows run at the same time and hit L2, which is worth
    // 6 % on the isolated contraction (1086 -> 1152 TFLOP/s sustained, 0.91 -> 0.86 pJ/FLOP) and 2.5 % on the step.
    p.group_m = epi == EPI_OUT ? 2 : 16;
    static const int env_group_m = []() { const char* v = std::getenv("MECLIP_GROUP_M"); return v ? std::atoi(v) : 0; }();
    if (env_group_m > 0 && epi == EPI_OUT) p.group_m = env_group_m;
    // strips: tile ids inside a group of 16 m-tiles share their columns; the sums pass keeps column
    // partials in registers over a strip.  Shorter strips when there are few tiles per SM.
    p.strip_len = 1;
    if (MECLIP_STRIPS && epi == EPI_SUMS && p.col_sum != nullptr) {
        const long long per_sm = (long long)p.num_m_tiles * p.num_n_tiles / sm_count();
        p.strip_len = per_sm >= 64 ? 16 : per_sm >= 32 ? 8 : per_sm >= 16 ? 4 : per_sm >= 8 ? 2 : 1;
    }
    p.idesc = umma_idesc_bf16(BM, bn, a.mn_major ? 1 : 0, b.mn_major ? 1 : 0);
    p.bn_last = bn;
    p.idesc_last = p.idesc;
    if (epi == EPI_OUT) {      // narrower last column tile: only as many 32-column chunks as hold valid columns
        const long long rest = n - (long long)(p.num_n_tiles - 1) * bn;
        int last = (int)((rest + 31) / 32 * 32);
        if (b.mn_major || rest > MAX_BN) last = (int)((rest + 63) / 64 * 64);
        if (last < bn) {
            p.bn_last = last;
            p.idesc_last = umma_idesc_bf16(BM, last, a.mn_major ? 1 : 0, b.mn_major ? 1 : 0);
        }
    }
    if ((long long)p.num_m_tiles * p.num_n_tiles > 0x7fffffffLL) return fail(MECLIP_EINVAL, "too many tiles");
    // shared memory: [<= 1023 B alignment slack][stages][tail]; as many stages as fit, at least 2
    p.stage_bytes = A_STAGE_BYTES + bn * BK * 2;
    int stages = (SMEM_LIMIT - 1024 - tail_bytes(epi)) / p.stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    static const int env_max_stages = []() { const char* v = std::getenv("MECLIP_MAX_STAGES"); return v ? std::atoi(v) : 0; }();
    static const bool env_static = []() { const char* v = std::getenv("MECLIP_STATIC_SCHED"); return v && v[0] == '1'; }();
    if (env_max_stages >= 2 && stages > env_max_stages) stages = env_max_stages;
    if (env_static) p.tile_counter = nullptr;
    if (stages < 2) return fail(MECLIP_EINVAL, "tile does not fit shared memory");
    if (pair) p.num_m_tiles = (int)((m + PAIR_BM - 1) / PAIR_BM);
    if (epi == EPI_OUT && p.bn_last < bn && p.num_n_tiles >= 2) {
        // Narrow tiles last (MECLIP_NARROW_LAST: 0 never (the default), 1 when the launch has fewer than four
        // waves of tiles, 2 always): the short tiles would even out the last wave, but they then read their
        // rows of the A operand a second time from HBM instead of from L2 next to the wide tiles of the same
        // rows.  Measured at B = 32768, D = 1152: dY alone 977 (off) / 971 (on) TFLOP/s, step 8.10-8.14 /
        // 8.24-8.27 ms (fewer than four waves), 8.40 ms (always).  Kept as a switch for that A/B only.
        static const int env_narrow = []() { const char* v = std::getenv("MECLIP_NARROW_LAST"); return v ? std::atoi(v) : 0; }();
        const long long slots = pair ? sm_count() / 2 : sm_count();
        const long long tiles_all = (long long)p.num_m_tiles * p.num_n_tiles;
        if (env_narrow == 2 || (env_narrow == 1 && tiles_all < 4 * slots)) p.narrow_last = 1;
    }
    if (pair) {
        const int amn = a.mn_major ? 1 : 0;
        p.wide = wide ? 1 : 0;
        p.idesc = umma_idesc_bf16(PAIR_BM, bn < MAX_BN ? bn : MAX_BN, amn, 0);
        p.idesc2 = wide ? umma_idesc_bf16(PAIR_BM, bn - MAX_BN, amn, 0) : 0u;
        p.idesc_last = umma_idesc_bf16(PAIR_BM, p.bn_last < MAX_BN ? p.bn_last : MAX_BN, amn, 0);
        p.idesc2_last = p.bn_last > MAX_BN ? umma_idesc_bf16(PAIR_BM, p.bn_last - MAX_BN, amn, 0) : 0u;
        p.stage_bytes = A_STAGE_BYTES + (bn / 2) * BK * 2;
        stages = (SMEM_LIMIT - 1024 - tail_bytes(epi)) / p.stage_bytes;
        if (stages > MAX_STAGES) stages = MAX_STAGES;
        if (env_max_stages >= 2 && stages > env_max_stages) stages = env_max_stages;
        p.num_stages = stages;
        const size_t pair_smem = 1024 + (size_t)stages * p.stage_bytes + tail_bytes(epi);
        if (f32) {
            p.idesc = p.idesc_last = umma_idesc_tf32(PAIR_BM, bn);
            if (epi == EPI_SUMS) return launch_pair_t<EPI_SUMS, 0, true>(ta, tb, tc, p, pair_smem, stream);
            return launch_pair_t<EPI_COEF, 0, true>(ta, tb, tc, p, pair_smem, stream);
        }
        if (epi == EPI_SUMS) return launch_pair_t<EPI_SUMS, 0>(ta, tb, tc, p, pair_smem, stream);
        if (epi == EPI_COEF) return launch_pair_t<EPI_COEF, 0>(ta, tb, tc, p, pair_smem, stream);
        if (epi == EPI_OUT) return a.mn_major ? launch_pair_t<EPI_OUT, 1>(ta, tb, tc, p, pair_smem, stream)
                                              : launch_pair_t<EPI_OUT, 0>(ta, tb, tc, p, pair_smem, stream);
        return fail(MECLIP_EINVAL, "unknown epilogue %d", epi);
    }
    p.num_stages = stages;
    const size_t smem_bytes = 1024 + (size_t)stages * p.stage_bytes + tail_bytes(epi);
#define MECLIP_DISPATCH(E)                                                                                        \
    if (epi == E) {                                                                                               \
        if (!a.mn_major && !b.mn_major) return launch_gemm_t<E, false, false>(ta, tb, tc, p, smem_bytes, stream); \
        if (!a.mn_major && b.mn_major) return launch_gemm_t<E, false, true>(ta, tb, tc, p, smem_bytes, stream);   \
        if (a.mn_major && b.mn_major) return launch_gemm_t<E, true, true>(ta, tb, tc, p, smem_bytes, stream);     \
        return launch_gemm_t<E, true, false>(ta, tb, tc, p, smem_bytes, stream);                                  \
    }
    if (epi == EPI_SUMS) return launch_gemm_t<EPI_SUMS, false, false>(ta, tb, tc, p, smem_bytes, stream);
    if (epi == EPI_COEF) return launch_gemm_t<EPI_COEF, false, false>(ta, tb, tc, p, smem_bytes, stream);
    MECLIP_DISPATCH(EPI_OUT)
#undef MECLIP_DISPATCH
    return fail(MECLIP_EINVAL, "unknown epilogue %d", epi);
}

// MECLIP_DUAL=0 launches the two contractions of a block separately (A/B switch).
static bool dual_allowed() {
    static const bool on = []() { const char* v = std::getenv("MECLIP_DUAL"); return !(v && v[0] == '0'); }();
    return on;
}

// Both contractions of one block of the backward in ONE launch of the CTA-pair kernel:
//   problem 0  dY [cols x n] (+)= G^T X   A = the panel read MN-major (M = cols, K = rows), B = X^T (K-major)
//   problem 1  dX [rows x n] (+)= G Y     A = the panel read K-major  (M = rows, K = cols), B = Y^T (K-major)
// Twice the tiles per launch means a fuller last wave (640 tiles instead of 2 x 320 on 74 CTA pairs) and one
// launch less per block.  py / px carry the outputs (out, ld_out, out_bf16, acc_in, ld_acc, tile_counter, status).
static int launch_contractions_dual(const void* panel, long long panel_rows_alloc, long long panel_chunks_alloc,
                                    const void* xt, long long ld_xt, const void* yt, long long ld_yt, long long rows,
                                    long long cols, long long n, const GemmParams& py, const GemmParams& px,
                                    cudaStream_t stream) {
    if (rows < 1 || cols < 1 || n < 1 || rows > 0x7fffffffLL || cols > 0x7fffffffLL) return fail(MECLIP_EINVAL, "dual contraction: bad extents");
    const int bn = 256;
    CUtensorMap tay, tby, tax, tbx;
    int rc = make_tmap_blocked(&tay, panel, rows, (cols + 63) / 64, panel_rows_alloc, BK, panel_chunks_alloc);   // G^T: K = rows
    if (rc) return rc;
    rc = make_tmap_blocked(&tax, panel, rows, (cols + 63) / 64, panel_rows_alloc, BM, panel_chunks_alloc);        // G: M = rows
    if (rc) return rc;
    rc = make_tmap(&tby, xt, rows, n, ld_xt, BK, bn / 2);     // X^T [n][K = rows]
    if (rc) return rc;
    rc = make_tmap(&tbx, yt, cols, n, ld_yt, BK, bn / 2);     // Y^T [n][K = cols]
    if (rc) return rc;
    GemmParams p = py;
    p.a_blocked = 1;
    p.m = (int)cols; p.n = (int)n; p.k = (int)rows; p.bn = bn;
    p.num_m_tiles = (int)((cols + PAIR_BM - 1) / PAIR_BM);
    p.num_n_tiles = (int)((n + bn - 1) / bn);
    p.k_steps = (int)((rows + BK - 1) / BK);
    p.m2 = (int)rows;
    p.num_m_tiles2 = (int)((rows + PAIR_BM - 1) / PAIR_BM);
    p.k_steps2 = (int)((cols + BK - 1) / BK);
    p.out2 = px.out; p.ld_out2 = px.ld_out; p.out_bf16_2 = px.out_bf16; p.acc_in2 = px.acc_in; p.ld_acc2 = px.ld_acc;
    p.dual = 1;
    p.tiles0 = p.num_m_tiles * p.num_n_tiles;
    if ((long long)p.tiles0 + (long long)p.num_m_tiles2 * p.num_n_tiles > 0x7fffffffLL) return fail(MECLIP_EINVAL, "too many tiles");
    p.trace = nullptr; p.trace_capacity = 0;
    p.wait_limit_ns = wait_limit_ns();
    p.group_m = 2;
    static const int env_group_m = []() { const char* v = std::getenv("MECLIP_GROUP_M"); return v ? std::atoi(v) : 0; }();
    if (env_group_m > 0) p.group_m = env_group_m;
    p.strip_len = 1;
    const long long rest = n - (long long)(p.num_n_tiles - 1) * bn;
    p.bn_last = (int)((rest + 31) / 32 * 32);
    p.idesc = umma_idesc_bf16(PAIR_BM, bn, 1, 0);
    p.idesc_last = umma_idesc_bf16(PAIR_BM, p.bn_last, 1, 0);
    p.idesc_p2 = umma_idesc_bf16(PAIR_BM, bn, 0, 0);
    p.idesc_last_p2 = umma_idesc_bf16(PAIR_BM, p.bn_last, 0, 0);
    p.wide = 0; p.idesc2 = 0; p.idesc2_last = 0; p.narrow_last = 0;
    static const bool env_static = []() { const char* v = std::getenv("MECLIP_STATIC_SCHED"); return v && v[0] == '1'; }();
    if (env_static) p.tile_counter = nullptr;
    p.stage_bytes = A_STAGE_BYTES + (bn / 2) * BK * 2;
    int stages = (SMEM_LIMIT - 1024 - tail_bytes(EPI_OUT)) / p.stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    static const int env_max_stages = []() { const char* v = std::getenv("MECLIP_MAX_STAGES"); return v ? std::atoi(v) : 0; }();
    if (env_max_stages >= 2 && stages > env_max_stages) stages = env_max_stages;
    p.num_stages = stages;
    const size_t smem = 1024 + (size_t)stages * p.stage_bytes + tail_bytes(EPI_OUT);
    return launch_pair_t<EPI_OUT, 2>(tay, tby, tax, p, smem, stream, &tbx, 4.0 * (double)rows * (double)cols * (double)n);
}

// ------------------------------------------------------------------------------------
// backward blocking
// ------------------------------------------------------------------------------------
// Rows of G formed per block.  The two contractions of a block have (rows / 256) x column tiles (dX) and
// (panel width / 256) x column tiles (dY) CTA-pair tiles, so a square block gives both the same number of
// tiles.  Measured at B = 32768, D = 1152, kernels timed alone (TFLOP/s dX / dY) and the step (ms), one GPU,
// one call: blocks of 32768 x 8192: 1205 / 977, 8.10-8.14; 16384 x 16384: 1141-1150 / 1136-1144, 8.03-8.13;
// with 1 GiB panels 32768 x 16384: 1254 / 1162, 8.07 and 16384 x 32768: 1173 / 1260, 7.98.
static constexpr long long ROW_BLOCK = 16384;
static constexpr long long PANEL_BYTES = 512ll << 20;          // most bytes one bf16 coefficient panel may take

struct GradPlan {
    long long row_block, panel_w, ldg;
    long long n_row_blocks, n_panels, n_blocks;
    int g_buffers;                       // 2 when there is more than one block: panel t+1 is formed while t is contracted
    size_t g_bytes, dx_bytes, dy_bytes, counter_bytes;
    long long ld_xt, ld_yt;              // pitches of the transposed operand copies X^T [d x rows], Y^T [d x cols]
    size_t xt_bytes, yt_bytes;
    size_t total() const { return g_bytes * g_buffers + dx_bytes + dy_bytes + counter_bytes + xt_bytes + yt_bytes; }
};

// test hook: smaller blocks so that small problems exercise the multi-block paths (0 = defaults)
static long long g_row_block_override = 0, g_panel_bytes_override = 0;

// A/B switches: MECLIP_ROW_BLOCK (rows, a multiple of 128) and MECLIP_PANEL_MIB change the built-in blocking
// for the whole process (the test hook above takes precedence).
static long long env_ll(const char* name) {
    const char* v = std::getenv(name);
    return v ? std::atoll(v) : 0;
}

// honour_overrides == false: the built-in constants, whatever the test hook or the environment say
// (meclip_grad_static promises a plan that fits its fixed scratch).
static GradPlan plan_grad(long long rows, long long cols, long long d, bool transposed_copies = true,
                          bool honour_overrides = true) {
    GradPlan g;
    static const long long env_row_block = env_ll("MECLIP_ROW_BLOCK") / 128 * 128;
    static const long long env_panel_bytes = env_ll("MECLIP_PANEL_MIB") << 20;
    long long row_block_max = ROW_BLOCK, panel_bytes = PANEL_BYTES;
    if (honour_overrides) {
        if (env_row_block > 0) row_block_max = env_row_block;
        if (env_panel_bytes > 0) panel_bytes = env_panel_bytes;
        if (g_row_block_override > 0) row_block_max = g_row_block_override;
        if (g_panel_bytes_override > 0) panel_bytes = g_panel_bytes_override;
    }
    g.row_block = rows < row_block_max ? rows : row_block_max;
    long long w = panel_bytes / (g.row_block * 2) / 256 * 256;
    if (w < 256) w = 256;
    if (w > 32768) w = 32768;
    if (w > cols) w = cols;
    g.panel_w = w;
    g.ldg = (long long)round_up((size_t)w, 64);
    g.n_row_blocks = (rows + g.row_block - 1) / g.row_block;
    g.n_panels = (cols + w - 1) / w;
    g.n_blocks = g.n_row_blocks * g.n_panels;
    g.g_buffers = g.n_blocks > 1 ? 2 : 1;
    g.g_bytes = round_up((size_t)g.row_block * g.ldg * 2, 256);
    g.dx_bytes = g.n_panels > 1 ? round_up((size_t)g.row_block * d * 4, 256) : 0;
    g.dy_bytes = g.n_row_blocks > 1 ? round_up((size_t)cols * d * 4, 256) : 0;
    g.counter_bytes = round_up((size_t)g.n_blocks * 3 * sizeof(unsigned int), 256);   // one tile counter per launch
    g.ld_xt = (long long)round_up((size_t)rows, 8);
    g.ld_yt = (long long)round_up((size_t)cols, 8);
    g.xt_bytes = transposed_copies ? round_up((size_t)d * g.ld_xt * 2, 256) : 0;
    g.yt_bytes = transposed_copies ? round_up((size_t)d * g.ld_yt * 2, 256) : 0;
    return g;
}

// ------------------------------------------------------------------------------------
// side streams: the two contractions of a block and the next block's coefficient pass
// run next to each other, so the tail of one kernel is filled by the next
// ------------------------------------------------------------------------------------
struct SideStreams {
    bool ready = false;
    cudaStream_t sx = nullptr, sy = nullptr;
    cudaEvent_t coef[2] = {nullptr, nullptr}, dx[2] = {nullptr, nullptr}, dy[2] = {nullptr, nullptr};
    cudaEvent_t join_x = nullptr, join_y = nullptr, fork = nullptr;
    std::mutex mutex;       // one meclip_grad enqueue at a time per device: the events are shared
};
static SideStreams g_side[64];
static std::mutex g_side_init_mutex;

static int get_side_streams(SideStreams** out) {
    int dev = 0;
    MECLIP_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MECLIP_EUNSUPPORTED, "device index %d out of range", dev);
    SideStreams& ss = g_side[dev];
    std::lock_guard<std::mutex> lock(g_side_init_mutex);
    if (!ss.ready) {
        MECLIP_CUDA(cudaStreamCreateWithFlags(&ss.sx, cudaStreamNonBlocking));
        MECLIP_CUDA(cudaStreamCreateWithFlags(&ss.sy, cudaStreamNonBlocking));
        cudaEvent_t* evs[9] = {&ss.coef[0], &ss.coef[1], &ss.dx[0], &ss.dx[1], &ss.dy[0], &ss.dy[1], &ss.join_x, &ss.join_y,
                               &ss.fork};
        for (auto e : evs) MECLIP_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        ss.ready = true;
    }
    *out = &ss;
    return MECLIP_OK;
}

static bool transposes_allowed() {
    static const bool off = []() { const char* v = std::getenv("MECLIP_NO_TRANSPOSE"); return v && v[0] == '1'; }();
    return !off;
}

static bool overlap_allowed() {
    static const bool env_serial = []() {
        const char* v = std::getenv("MECLIP_SERIAL");
        return v != nullptr && v[0] != '\0' && v[0] != '0';
    }();
    if (env_serial) return false;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    return !g_prof_on;      // per-kernel timing wants kernels that do not share the GPU
}

static int check_out_mode(int mode) { return mode == MECLIP_STORE_BF16 || mode == MECLIP_STORE_F32 || mode == MECLIP_ACCUM_F32; }

// fp32 operand for the tf32 passes: out[r, c] = tf32(x[r, c] * inv[r]) (inv == nullptr: x itself), zeros in the pad
// columns.  Rounded to nearest here (cvt.rna.tf32), because the tensor cores just drop the 13 low mantissa bits
// of what they read: with pre-rounded operands that truncation changes nothing and the products are unbiased.
__global__ void __launch_bounds__(ROW_KERNEL_THREADS)
operand_f32_kernel(const float* __restrict__ x, long long ldx, long long rows, int d, int dpad,
                   const float* __restrict__ inv, float* __restrict__ out, long long ldo) {
    const long long row = (long long)blockIdx.x * (ROW_KERNEL_THREADS / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float f = inv != nullptr ? inv[row] : 1.f;
    const float* xr = x + row * ldx;
    float* o = out + row * ldo;
    for (int c = lane; c < dpad; c += 32) {
        uint32_t bits = 0u;
        if (c < d) {
            const float v = xr[c] * f;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(v));
        }
        o[c] = __uint_as_float(bits);
    }
}

}  // namespace meclip

using namespace meclip;

// ------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------
extern "C" {

int meclip_version(void) { return 100; }

const char* meclip_status_string(int code) {
    switch (code) {
        case MECLIP_OK: return "ok";
        case MECLIP_EINVAL: return "invalid argument";
        case MECLIP_ENOSPC: return "workspace too small";
        case MECLIP_ECUDA: return "CUDA error";
        case MECLIP_ETIMEOUT: return "bounded wait inside a kernel expired";
        case MECLIP_EUNSUPPORTED: return "unsupported device or driver";
        default: return "unknown status";
    }
}

int meclip_last_error(char* buf, size_t buf_len) {
    if (buf == nullptr || buf_len == 0) return MECLIP_EINVAL;
    std::lock_guard<std::mutex> lock(g_err_mutex);
    std::strncpy(buf, g_last_error.c_str(), buf_len - 1);
    buf[buf_len - 1] = '\0';
    return MECLIP_OK;
}

int meclip_read_status(const int* status, void* stream) {
    if (status == nullptr) return fail(MECLIP_EINVAL, "status pointer is null");
    int host = 0;
    MECLIP_CUDA(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MECLIP_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (host != 0) return fail(MECLIP_ETIMEOUT, "a kernel gave up waiting on a barrier (status word %d)", host);
    return MECLIP_OK;
}

int meclip_debug_set_blocking(int64_t row_block, int64_t panel_bytes) {
    if (row_block < 0 || panel_bytes < 0 || (row_block > 0 && row_block % 128 != 0))
        return fail(MECLIP_EINVAL, "debug_set_blocking: row_block must be a multiple of 128");
    g_row_block_override = row_block;
    g_panel_bytes_override = panel_bytes;
    return MECLIP_OK;
}

int meclip_debug_set_trace(void* device_words, size_t n_words) {
    if (device_words == nullptr || n_words < 5) { g_trace_buf = nullptr; g_trace_capacity = 0; return MECLIP_OK; }
    g_trace_buf = reinterpret_cast<unsigned long long*>(device_words);
    g_trace_capacity = (unsigned int)((n_words - 2) / 3);
    return MECLIP_OK;
}

long long meclip_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int meclip_profile_begin(void) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    for (auto& r : g_prof) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
    g_prof.clear();
    g_prof_on = true;
    return MECLIP_OK;
}

int meclip_profile_end(double* ms_by_tag, long long* launches_by_tag, double* flops_by_tag, int n_tags) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_on = false;
    for (int i = 0; i < n_tags; ++i) {
        if (ms_by_tag) ms_by_tag[i] = 0.0;
        if (launches_by_tag) launches_by_tag[i] = 0;
        if (flops_by_tag) flops_by_tag[i] = 0.0;
    }
    int rc = MECLIP_OK;
    for (auto& r : g_prof) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.stop) != cudaSuccess || cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess)
            rc = MECLIP_ECUDA;
        if (r.tag >= 0 && r.tag < n_tags) {
            if (ms_by_tag) ms_by_tag[r.tag] += ms;
            if (launches_by_tag) launches_by_tag[r.tag] += 1;
            if (flops_by_tag) flops_by_tag[r.tag] += r.flops;
        }
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    g_prof.clear();
    if (rc) return fail(rc, "profile_end: reading an event failed");
    return MECLIP_OK;
}

int meclip_accumulate_f32(float* dst, const float* src, int64_t n, void* stream) {
    if (dst == nullptr || src == nullptr || n < 0 || n % 4 != 0 || !aligned16(dst) || !aligned16(src))
        return fail(MECLIP_EINVAL, "accumulate_f32: need 16-byte aligned pointers and n a multiple of 4");
    if (n == 0) return MECLIP_OK;
    const long long n4 = n / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
    ScopedTiming timing((cudaStream_t)stream, TAG_ACCUM, 12.0 * (double)n);
    accumulate_f32_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dst, src, n4);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_accumulate_many_f32(float* dst, const float* src, int n_src, int64_t src_stride, int64_t n, void* stream) {
    if (dst == nullptr || src == nullptr || n_src < 1 || n < 0 || n % 4 != 0 || src_stride % 4 != 0 || src_stride < n ||
        !aligned16(dst) || !aligned16(src))
        return fail(MECLIP_EINVAL, "accumulate_many_f32: need 16-byte aligned pointers, n and stride multiples of 4, stride >= n");
    if (n == 0) return MECLIP_OK;
    const long long n4 = n / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
    ScopedTiming timing((cudaStream_t)stream, TAG_ACCUM, 4.0 * (double)n * (n_src + 2));
    accumulate_many_f32_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dst, src, n_src, src_stride / 4, n4);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_normalize_fwd(const void* x, int x_dtype, int64_t rows, int64_t d, int64_t ldx, int normalize,
                         void* x_hat_bf16, int64_t ldh, float* inv_norm, void* stream) {
    if (x == nullptr || x_hat_bf16 == nullptr) return fail(MECLIP_EINVAL, "normalize_fwd: null pointer");
    const int64_t dpad = (d + 7) / 8 * 8;
    if (rows < 1 || d < 1 || ldx < d || ldh < dpad) return fail(MECLIP_EINVAL, "normalize_fwd: need rows, d >= 1, ldx >= d, ldh >= round_up(d, 8)");
    if (!aligned16(x_hat_bf16) || ldh % 8 != 0)
        return fail(MECLIP_EINVAL, "normalize_fwd: x_hat must be 16-byte aligned with a pitch that is a multiple of 8");
    if (normalize && inv_norm == nullptr) return fail(MECLIP_EINVAL, "normalize_fwd: inv_norm is null");
    const int elt = x_dtype == MECLIP_F32 ? 4 : 2;
    const int vec = (d % 8 == 0) && aligned16(x) && ((ldx * elt) % 16 == 0);
    const int wpb = ROW_KERNEL_THREADS / 32;
    const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
    cudaStream_t s = (cudaStream_t)stream;
    ScopedTiming timing(s, TAG_NORM_FWD, (double)rows * ((double)d * elt + (double)dpad * 2 + (normalize ? 4 : 0)));
    __nv_bfloat16* out = (__nv_bfloat16*)x_hat_bf16;
    if (x_dtype == MECLIP_F32)
        normalize_fwd_kernel<float><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const float*)x, ldx, rows, (int)d, (int)dpad, normalize, vec, out, ldh, inv_norm);
    else if (x_dtype == MECLIP_BF16)
        normalize_fwd_kernel<__nv_bfloat16><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const __nv_bfloat16*)x, ldx, rows, (int)d, (int)dpad, normalize, vec, out, ldh, inv_norm);
    else if (x_dtype == MECLIP_F16)
        normalize_fwd_kernel<__half><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const __half*)x, ldx, rows, (int)d, (int)dpad, normalize, vec, out, ldh, inv_norm);
    else
        return fail(MECLIP_EINVAL, "normalize_fwd: bad dtype %d", x_dtype);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

}  // extern "C"

namespace {
template <typename TG>
int launch_normalize_bwd(const TG* g, int64_t ldg, const __nv_bfloat16* xh, int64_t ldh, const float* inv_norm, int64_t rows,
                         int64_t d, void* dx, int dx_dtype, int64_t lddx, int vec_out, unsigned grid, cudaStream_t s) {
    if (dx_dtype == MECLIP_F32)
        normalize_bwd_kernel<TG, float><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g, ldg, xh, ldh, inv_norm, rows, (int)d, vec_out, (float*)dx, lddx);
    else if (dx_dtype == MECLIP_BF16)
        normalize_bwd_kernel<TG, __nv_bfloat16><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g, ldg, xh, ldh, inv_norm, rows, (int)d, vec_out, (__nv_bfloat16*)dx, lddx);
    else if (dx_dtype == MECLIP_F16)
        normalize_bwd_kernel<TG, __half><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g, ldg, xh, ldh, inv_norm, rows, (int)d, vec_out, (__half*)dx, lddx);
    else
        return fail(MECLIP_EINVAL, "normalize_bwd: bad output dtype %d", dx_dtype);
    return MECLIP_OK;
}
}  // namespace

extern "C" {

int meclip_normalize_bwd(const void* g, int g_dtype, int64_t ldg, const void* x_hat_bf16, int64_t ldh,
                         const float* inv_norm, int64_t rows, int64_t d, void* dx, int dx_dtype, int64_t lddx,
                         void* stream) {
    if (g == nullptr || dx == nullptr || (inv_norm != nullptr && x_hat_bf16 == nullptr))
        return fail(MECLIP_EINVAL, "normalize_bwd: null pointer");
    const int64_t dpad = (d + 7) / 8 * 8;
    if (rows < 1 || d < 1 || ldg < dpad || (x_hat_bf16 != nullptr && ldh < dpad) || lddx < d)
        return fail(MECLIP_EINVAL, "normalize_bwd: need rows, d >= 1, ldg and ldh >= round_up(d, 8), lddx >= d");
    if (!aligned16(g) || (x_hat_bf16 != nullptr && !aligned16(x_hat_bf16)) || ldg % 8 != 0 || (x_hat_bf16 != nullptr && ldh % 8 != 0))
        return fail(MECLIP_EINVAL, "normalize_bwd: g and x_hat must be 16-byte aligned with pitches multiples of 8");
    const int oelt = dx_dtype == MECLIP_F32 ? 4 : 2;
    const int vec_out = (d % 8 == 0) && aligned16(dx) && ((lddx * oelt) % 16 == 0);
    const int wpb = ROW_KERNEL_THREADS / 32;
    const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
    cudaStream_t s = (cudaStream_t)stream;
    ScopedTiming timing(s, TAG_NORM_BWD, (double)rows * ((double)dpad * ((g_dtype == MECLIP_F32 ? 4 : 2) + (inv_norm ? 2 : 0)) +
                                                       (double)d * oelt + (inv_norm ? 4 : 0)));
    const __nv_bfloat16* xh = (const __nv_bfloat16*)x_hat_bf16;
    int rc;
    if (g_dtype == MECLIP_F32) rc = launch_normalize_bwd<float>((const float*)g, ldg, xh, ldh, inv_norm, rows, d, dx, dx_dtype, lddx, vec_out, grid, s);
    else if (g_dtype == MECLIP_BF16) rc = launch_normalize_bwd<__nv_bfloat16>((const __nv_bfloat16*)g, ldg, xh, ldh, inv_norm, rows, d, dx, dx_dtype, lddx, vec_out, grid, s);
    else return fail(MECLIP_EINVAL, "normalize_bwd: bad dtype %d", g_dtype);
    if (rc) return rc;
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

}  // extern "C"

namespace meclip {
struct DetLayout { int row_slots, col_slots; long long ld_rows, ld_cols; size_t col_off, total; };
static DetLayout det_layout(int64_t rows, int64_t cols) {
    DetLayout l;
    const int bn = pick_bn(cols);
    l.row_slots = 2 * (int)((cols + bn - 1) / bn);
    l.col_slots = (int)((rows + 127) / 128);
    l.ld_rows = (long long)round_up((size_t)rows, 64);
    l.ld_cols = (long long)round_up((size_t)cols, 64);
    l.col_off = round_up((size_t)l.row_slots * l.ld_rows * 4, 256);
    l.total = l.col_off + round_up((size_t)l.col_slots * l.ld_cols * 4, 256);
    return l;
}

static int sum_exp_impl(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                        int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                        float* col_sum, float* diag_s, unsigned int* tile_counter, int* status, void* stream,
                        const DeviceScalars& ds, void* det_ws = nullptr, size_t det_ws_bytes = 0, bool f32 = false) {
    // f32: x and y are fp32 matrices (same shape rules), multiplied as tf32
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT) return fail(MECLIP_EINVAL, "sum_exp: bad kind %d", kind);
    if (x_bf16 == nullptr || y_bf16 == nullptr || row_sum == nullptr || diag_s == nullptr)
        return fail(MECLIP_EINVAL, "sum_exp: null pointer");
    if (kind == MECLIP_CLIP && col_sum == nullptr) return fail(MECLIP_EINVAL, "sum_exp: CLIP needs col_sum");
    if (rows < 1 || cols < 1 || d < 8 || d % 8 != 0 || ldx < d || ldy < d)
        return fail(MECLIP_EINVAL, "sum_exp: need rows, cols >= 1, d a multiple of 8 (got %lld), ld >= d", (long long)d);
    if (ds.t == nullptr && !(temperature > 0.f)) return fail(MECLIP_EINVAL, "sum_exp: temperature must be positive");
    int rc = check_device();
    if (rc) return rc;
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.fmul = 1.4426950408889634f / temperature;
    p.fadd = -p.fmul;
    p.t_dev = ds.t;
    p.diag_shift = (long long)row_off - (long long)col_off;
    p.row_sum = row_sum;
    p.col_sum = (kind == MECLIP_CLIP) ? col_sum : nullptr;
    p.diag = diag_s;
    p.tile_counter = tile_counter;
    p.status = status;
    Operand a{x_bf16, ldx, false, 0, f32}, b{y_bf16, ldy, false, 0, f32};
    t_tag = TAG_SUMS;
    const int bn = pick_bn(cols);
    if (det_ws == nullptr) return launch_gemm(EPI_SUMS, a, b, rows, cols, d, bn, p, (cudaStream_t)stream);
    // Deterministic sums: every partial goes to its own slot (plain stores), a second kernel adds the slots in a
    // fixed order.  Slots: 2 per column tile for the rows, 1 per 128 rows for the columns.
    if (!MECLIP_STRIPS) return fail(MECLIP_EUNSUPPORTED, "deterministic sums need the default epilogue build");
    const DetLayout l = det_layout(rows, cols);
    if ((reinterpret_cast<uintptr_t>(det_ws) & 255u) != 0 || det_ws_bytes < l.total)
        return fail(MECLIP_ENOSPC, "sum_exp_det: workspace %zu < %zu bytes or not 256-byte aligned", det_ws_bytes, l.total);
    cudaStream_t s = (cudaStream_t)stream;
    MECLIP_CUDA(cudaMemsetAsync(det_ws, 0, l.total, s));      // slots no tile writes (ragged edges) count as zero
    p.row_part = reinterpret_cast<float*>(det_ws);
    p.part_ld_rows = l.ld_rows;
    p.col_part = kind == MECLIP_CLIP ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(det_ws) + l.col_off) : nullptr;
    p.part_ld_cols = l.ld_cols;
    rc = launch_gemm(EPI_SUMS, a, b, rows, cols, d, bn, p, s);
    if (rc) return rc;
    {
        ScopedTiming timing(s, TAG_ROW, 4.0 * (double)rows * (l.row_slots + 2));
        reduce_parts_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(p.row_part, l.row_slots, l.ld_rows, rows, row_sum);
    }
    if (p.col_part != nullptr) {
        ScopedTiming timing(s, TAG_ROW, 4.0 * (double)cols * (l.col_slots + 2));
        reduce_parts_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, s>>>(p.col_part, l.col_slots, l.ld_cols, cols, col_sum);
    }
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

static int loss_finalize_impl(int kind, const float* row_sum, const float* col_sum, const float* diag_s, int64_t n,
                              float temperature, float scale, int accumulate, float* loss_out, void* stream,
                              const DeviceScalars& ds) {
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT) return fail(MECLIP_EINVAL, "loss_finalize: bad kind %d", kind);
    if (row_sum == nullptr || diag_s == nullptr || loss_out == nullptr || n < 1 || (ds.t == nullptr && !(temperature > 0.f)))
        return fail(MECLIP_EINVAL, "loss_finalize: bad argument");
    if (kind == MECLIP_CLIP && col_sum == nullptr) return fail(MECLIP_EINVAL, "loss_finalize: CLIP needs col_sum");
    ScopedTiming timing((cudaStream_t)stream, TAG_ROW, (double)n * (kind == MECLIP_CLIP ? 12.0 : 8.0));
    loss_finalize_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(row_sum, kind == MECLIP_CLIP ? col_sum : nullptr, diag_s, n,
                                                               1.f / temperature, ds.t, scale, accumulate, loss_out);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}
}  // namespace meclip

extern "C" {

int meclip_bind_device_scalars(const float* temperature_or_scale, const float* logit_bias, int grad_scale_rule) {
    if (grad_scale_rule < 0 || grad_scale_rule > 3) return fail(MECLIP_EINVAL, "bind_device_scalars: bad rule %d", grad_scale_rule);
    t_scalars.t = temperature_or_scale;
    t_scalars.b = logit_bias;
    t_scalars.g_rule = temperature_or_scale != nullptr ? grad_scale_rule : 0;
    return MECLIP_OK;
}

int meclip_sum_exp(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                   int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                   float* col_sum, float* diag_s, unsigned int* tile_counter, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    NvtxRange range("meclip_sum_exp");
    return sum_exp_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                        diag_s, tile_counter, status, stream, ds);
}

int meclip_operand_f32(const float* x, int64_t rows, int64_t d, int64_t ldx, const float* inv_norm, float* out,
                       int64_t ldo, void* stream) {
    if (x == nullptr || out == nullptr) return fail(MECLIP_EINVAL, "operand_f32: null pointer");
    const int64_t dpad = (d + 7) / 8 * 8;
    if (rows < 1 || d < 1 || ldx < d || ldo < dpad || ldo % 4 != 0 || !aligned16(out))
        return fail(MECLIP_EINVAL, "operand_f32: need rows, d >= 1, ldx >= d, ldo >= round_up(d, 8), out 16-byte aligned");
    const int wpb = ROW_KERNEL_THREADS / 32;
    ScopedTiming timing((cudaStream_t)stream, TAG_NORM_FWD, (double)rows * ((double)d * 4 + (double)dpad * 4));
    operand_f32_kernel<<<(unsigned)((rows + wpb - 1) / wpb), ROW_KERNEL_THREADS, 0, (cudaStream_t)stream>>>(
        x, ldx, rows, (int)d, (int)dpad, inv_norm, out, ldo);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_sum_exp_tf32(int kind, const float* x_f32, const float* y_f32, int64_t rows, int64_t cols, int64_t d,
                        int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                        float* col_sum, float* diag_s, unsigned int* tile_counter, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    NvtxRange range("meclip_sum_exp_tf32");
    return sum_exp_impl(kind, x_f32, y_f32, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                        diag_s, tile_counter, status, stream, ds, nullptr, 0, true);
}

size_t meclip_sum_exp_det_workspace_bytes(int64_t rows, int64_t cols) {
    if (rows < 1 || cols < 1) return 0;
    return det_layout(rows, cols).total;
}

int meclip_sum_exp_det(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                       int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                       float* col_sum, float* diag_s, unsigned int* tile_counter, void* workspace,
                       size_t workspace_bytes, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (workspace == nullptr) return fail(MECLIP_EINVAL, "sum_exp_det: workspace is null");
    NvtxRange range("meclip_sum_exp_det");
    return sum_exp_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                        diag_s, tile_counter, status, stream, ds, workspace, workspace_bytes);
}

int meclip_loss_finalize(int kind, const float* row_sum, const float* col_sum, const float* diag_s, int64_t n,
                         float temperature, float scale, int accumulate, float* loss_out, void* stream) {
    const DeviceScalars ds = take_scalars();
    return loss_finalize_impl(kind, row_sum, col_sum, diag_s, n, temperature, scale, accumulate, loss_out, stream, ds);
}

size_t meclip_grad_workspace_bytes(int64_t rows, int64_t cols, int64_t d) {
    if (rows < 1 || cols < 1 || d < 1) return 0;
    return plan_grad(rows, cols, d, true).total() + 256;
}

}  // extern "C"

namespace meclip {

// The backward over one rows x cols block.  overlap == false keeps every launch on the caller's
// stream and creates no stream or event.
static int grad_impl(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                     int64_t ldy, float temperature, int64_t row_off, int64_t col_off, const float* row_sum,
                     const float* col_sum, const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx,
                     void* dy, int dy_mode, int64_t lddy, void* workspace, size_t workspace_bytes, int* status,
                     cudaStream_t s0, bool overlap, bool transposed_copies, float* sg_acc = nullptr,
                     float logit_scale = 0.f, float logit_bias = 0.f, int64_t n_extra = 0, bool plain_e = false,
                     const DeviceScalars& ds = DeviceScalars(), bool honour_overrides = true,
                     const float* x_f32 = nullptr, int64_t ldxf = 0, const float* y_f32 = nullptr, int64_t ldyf = 0) {
    // x_f32 / y_f32: optional fp32 copies of the operands; the coefficient pass then forms S from them with tf32
    // MMAs (the contractions keep the bf16 operands)
    NvtxRange range("meclip_grad");
    if ((x_f32 == nullptr) != (y_f32 == nullptr) || (x_f32 != nullptr && (ldxf < d || ldyf < d)))
        return fail(MECLIP_EINVAL, "grad: fp32 operands come as a pair with pitches >= d");
    // kind MECLIP_SIGLIP: `temperature` is unused, the element function is sigmoid(logit_scale * s + logit_bias),
    // there are no row / column sums and both inputs get a gradient
    // plain_e (LiT only): the panel holds E itself (no 1/r, no diagonal term) and the contraction runs over
    // d + n_extra columns of Y, whose column d is all ones: dx receives [E Y | row sums of E | 0 ...]
    const bool siglip = (kind == MECLIP_SIGLIP);
    const int64_t dn = d + n_extra;       // columns of the contraction outputs and of the transposed copies
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT && !siglip) return fail(MECLIP_EINVAL, "grad: bad kind %d", kind);
    if (x_bf16 == nullptr || y_bf16 == nullptr || (row_sum == nullptr && !siglip && !plain_e) || workspace == nullptr)
        return fail(MECLIP_EINVAL, "grad: null pointer");
    if (plain_e && (kind != MECLIP_LIT || n_extra < 0 || n_extra % 8 != 0)) return fail(MECLIP_EINVAL, "grad: bad fused-forward arguments");
    if (kind == MECLIP_CLIP && col_sum == nullptr) return fail(MECLIP_EINVAL, "grad: CLIP needs col_sum");
    if (kind == MECLIP_LIT) dy = nullptr;      // the second argument of LiT is frozen
    if (dx == nullptr && dy == nullptr) return fail(MECLIP_EINVAL, "grad: null pointer (no gradient output requested)");
    if (rows < 1 || cols < 1 || d < 8 || d % 8 != 0 || ldx < d || ldy < dn || (dx != nullptr && lddx < dn) || (dy != nullptr && lddy < d))
        return fail(MECLIP_EINVAL, "grad: need rows, cols >= 1, d a multiple of 8, ld >= d");
    if ((dx != nullptr && !check_out_mode(dx_mode)) || (dy != nullptr && !check_out_mode(dy_mode))) return fail(MECLIP_EINVAL, "grad: bad output mode");
    if ((dx != nullptr && (!aligned16(dx) || lddx % 8 != 0)) || (dy != nullptr && (!aligned16(dy) || lddy % 8 != 0)))
        return fail(MECLIP_EINVAL, "grad: outputs must be 16-byte aligned with pitches multiples of 8");
    const bool want_dx = dx != nullptr, want_dy = dy != nullptr;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(MECLIP_EINVAL, "grad: workspace must be 256-byte aligned");
    if (!siglip && ds.t == nullptr && !(temperature > 0.f)) return fail(MECLIP_EINVAL, "grad: temperature must be positive");
    int rc = check_device();
    if (rc) return rc;
    const GradPlan plan = plan_grad(rows, cols, dn, transposed_copies, honour_overrides);
    if (workspace_bytes < plan.total())
        return fail(MECLIP_ENOSPC, "grad: workspace %zu < %zu bytes", workspace_bytes, plan.total());
    const bool clip = (kind == MECLIP_CLIP);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    __nv_bfloat16* gpanel[2] = {reinterpret_cast<__nv_bfloat16*>(ws),
                                reinterpret_cast<__nv_bfloat16*>(ws + (plan.g_buffers > 1 ? plan.g_bytes : 0))};
    uint8_t* after_g = ws + plan.g_bytes * plan.g_buffers;
    float* dx_scratch = reinterpret_cast<float*>(after_g);
    float* dy_scratch = reinterpret_cast<float*>(after_g + plan.dx_bytes);
    unsigned int* counters = reinterpret_cast<unsigned int*>(after_g + plan.dx_bytes + plan.dy_bytes);
    __nv_bfloat16* xt = reinterpret_cast<__nv_bfloat16*>(after_g + plan.dx_bytes + plan.dy_bytes + plan.counter_bytes);
    __nv_bfloat16* yt = reinterpret_cast<__nv_bfloat16*>(after_g + plan.dx_bytes + plan.dy_bytes + plan.counter_bytes + plan.xt_bytes);
    const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(x_bf16);
    const __nv_bfloat16* Y = reinterpret_cast<const __nv_bfloat16*>(y_bf16);
    // wide tiles; a narrower last one takes the remainder (see pick_contraction_bn)
    const size_t dx_elt = dx_mode == MECLIP_STORE_BF16 ? 2 : 4;
    const size_t dy_elt = dy_mode == MECLIP_STORE_BF16 ? 2 : 4;

    SideStreams* side = nullptr;
    std::unique_lock<std::mutex> side_lock;
    cudaStream_t sx = s0, sy = s0;
    if (overlap) {
        rc = get_side_streams(&side);
        if (rc) return rc;
        side_lock = std::unique_lock<std::mutex>(side->mutex);
        sx = side->sx;
        sy = side->sy;
    }
    // both contractions of a block in one launch: needs both outputs, K-major B operands (the transposed copies)
    // and the 256-column CTA-pair tiles
    const bool use_dual = want_dx && want_dy && transposed_copies && dual_allowed() && pair_mode() != 0 && !wide_allowed() &&
                          dn == d && d >= 256 && g_trace_buf == nullptr;
    if (use_dual) sy = sx;      // one side stream carries the transposes and the contractions
    // the tile counters are the only part of the workspace that has to start at zero
    MECLIP_CUDA(cudaMemsetAsync(counters, 0, plan.counter_bytes, s0));
    if (transposed_copies) {
        // Y^T is only read by the dX contractions and X^T by the dY contractions, so with side streams
        // the transposes run there, under the first coefficient pass
        if (overlap) {
            MECLIP_CUDA(cudaEventRecord(side->fork, s0));
            if (want_dx) MECLIP_CUDA(cudaStreamWaitEvent(sx, side->fork, 0));
            if (want_dy) MECLIP_CUDA(cudaStreamWaitEvent(sy, side->fork, 0));
        }
        if (want_dx) {
            ScopedTiming timing(sx, TAG_TRANSPOSE, 4.0 * (double)cols * (double)dn);
            dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((dn + 63) / 64));
            transpose_bf16_kernel<<<grid, 256, 0, sx>>>(Y, ldy, cols, (int)dn, yt, plan.ld_yt);
        }
        if (want_dy) {
            ScopedTiming timing(sy, TAG_TRANSPOSE, 4.0 * (double)rows * (double)d);
            dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((d + 63) / 64));
            transpose_bf16_kernel<<<grid, 256, 0, sy>>>(X, ldx, rows, (int)d, xt, plan.ld_xt);
        }
        MECLIP_CUDA(cudaGetLastError());
    }

    long long t = 0;
    for (long long rb = 0; rb < plan.n_row_blocks; ++rb) {
        const long long r0 = rb * plan.row_block;
        const long long nr = (rows - r0) < plan.row_block ? (rows - r0) : plan.row_block;
        for (long long cp = 0; cp < plan.n_panels; ++cp, ++t) {
            const long long c0 = cp * plan.panel_w;
            const long long nc = (cols - c0) < plan.panel_w ? (cols - c0) : plan.panel_w;
            const int gb = (int)(t & 1) & (plan.g_buffers - 1);
            // (1) coefficient panel G [nr x nc] = epi(X[r0:] Y[c0:]^T), once its buffer is free again
            if (overlap && t >= 2) {
                if (want_dx) MECLIP_CUDA(cudaStreamWaitEvent(s0, side->dx[gb], 0));
                if (want_dy) MECLIP_CUDA(cudaStreamWaitEvent(s0, side->dy[gb], 0));
            }
            {
                GemmParams p;
                std::memset(&p, 0, sizeof(p));
                if (siglip) {
                    p.sigmoid = 1;
                    p.fmul = logit_scale * 1.4426950408889634f;
                    p.fadd = logit_bias * 1.4426950408889634f;
                } else {
                    p.fmul = 1.4426950408889634f / temperature;
                    p.fadd = -p.fmul;
                }
                p.diag_shift = ((long long)row_off + r0) - ((long long)col_off + c0);
                p.r = (siglip || plain_e) ? nullptr : row_sum + r0;
                p.c = clip ? col_sum + c0 : nullptr;
                p.grad_out = grad_out;
                p.coef = clip ? 0.5f * grad_scale : grad_scale;
                p.dcoef = plain_e ? 0.f : grad_scale;
                p.sg_acc = sg_acc;
                p.t_dev = ds.t;
                p.b_dev = ds.b;
                p.g_rule = ds.g_rule;
                p.tile_counter = counters + 3 * t;
                p.status = status;
                Operand a{X + r0 * ldx, ldx, false}, b{Y + c0 * ldy, ldy, false};
                if (x_f32 != nullptr) {
                    a = Operand{x_f32 + r0 * ldxf, ldxf, false, 0, true};
                    b = Operand{y_f32 + c0 * ldyf, ldyf, false, 0, true};
                }
                t_tag = TAG_COEF;
                rc = launch_gemm(EPI_COEF, a, b, nr, nc, d, pick_bn(nc), p, s0, gpanel[gb], plan.row_block, plan.ldg / 64);
                if (rc) return rc;
            }
            if (overlap) {
                MECLIP_CUDA(cudaEventRecord(side->coef[gb], s0));
                if (want_dx) MECLIP_CUDA(cudaStreamWaitEvent(sx, side->coef[gb], 0));
                if (want_dy) MECLIP_CUDA(cudaStreamWaitEvent(sy, side->coef[gb], 0));
            }
            // (3) dY[c0:] (+)= G^T X[r0:]        M = nc, N = d, K = nr; A = G^T (M contiguous), B = X (N contiguous)
            //     issued before dX: its tiles are the long ones (K = nr)
            GemmParams py;
            std::memset(&py, 0, sizeof(py));
            if (want_dy) {
                GemmParams& p = py;
                p.status = status;
                p.tile_counter = counters + 3 * t + 2;
                uint8_t* user = reinterpret_cast<uint8_t*>(dy) + (size_t)c0 * lddy * dy_elt;
                float* scratch = dy_scratch + (size_t)c0 * d;
                if (dy_mode == MECLIP_ACCUM_F32) {
                    p.acc_in = reinterpret_cast<const float*>(user); p.ld_acc = lddy;
                    p.out = user; p.ld_out = lddy; p.out_bf16 = 0;
                } else if (plan.n_row_blocks == 1) {
                    p.out = user; p.ld_out = lddy; p.out_bf16 = (dy_mode == MECLIP_STORE_BF16);
                } else {
                    if (rb > 0) { p.acc_in = scratch; p.ld_acc = d; }
                    if (rb == plan.n_row_blocks - 1) { p.out = user; p.ld_out = lddy; p.out_bf16 = (dy_mode == MECLIP_STORE_BF16); }
                    else { p.out = scratch; p.ld_out = d; p.out_bf16 = 0; }
                }
                if (!use_dual) {
                    Operand a{gpanel[gb], plan.ldg / 64, true, plan.row_block}, b{X + r0 * ldx, ldx, true};
                    if (transposed_copies) b = Operand{xt + r0, plan.ld_xt, false};   // [d][K = rows] K-major
                    t_tag = TAG_DY;
                    rc = launch_gemm(EPI_OUT, a, b, nc, d, nr, pick_contraction_bn(nc, d, overlap, transposed_copies), p, sy);
                    if (rc) return rc;
                    if (overlap) MECLIP_CUDA(cudaEventRecord(side->dy[gb], sy));
                }
            }
            // (2) dX[r0:] (+)= G Y[c0:]          M = nr, N = d, K = nc; A = G (K contiguous), B = Y (N contiguous)
            if (want_dx) {
                GemmParams p;
                std::memset(&p, 0, sizeof(p));
                p.status = status;
                p.tile_counter = counters + 3 * t + 1;
                uint8_t* user = reinterpret_cast<uint8_t*>(dx) + (size_t)r0 * lddx * dx_elt;
                if (dx_mode == MECLIP_ACCUM_F32) {
                    p.acc_in = reinterpret_cast<const float*>(user); p.ld_acc = lddx;
                    p.out = user; p.ld_out = lddx; p.out_bf16 = 0;
                } else if (plan.n_panels == 1) {
                    p.out = user; p.ld_out = lddx; p.out_bf16 = (dx_mode == MECLIP_STORE_BF16);
                } else {
                    if (cp > 0) { p.acc_in = dx_scratch; p.ld_acc = dn; }
                    if (cp == plan.n_panels - 1) { p.out = user; p.ld_out = lddx; p.out_bf16 = (dx_mode == MECLIP_STORE_BF16); }
                    else { p.out = dx_scratch; p.ld_out = dn; p.out_bf16 = 0; }
                }
                if (use_dual) {
                    t_tag = TAG_DX;         // one launch: its time and FLOPs are booked under the dX tag
                    rc = launch_contractions_dual(gpanel[gb], plan.row_block, plan.ldg / 64, xt + r0, plan.ld_xt, yt + c0,
                                                  plan.ld_yt, nr, nc, d, py, p, sx);
                    if (rc) return rc;
                    if (overlap) {
                        MECLIP_CUDA(cudaEventRecord(side->dx[gb], sx));
                        MECLIP_CUDA(cudaEventRecord(side->dy[gb], sx));
                    }
                } else {
                    Operand a{gpanel[gb], plan.ldg / 64, false, plan.row_block}, b{Y + c0 * ldy, ldy, true};
                    if (transposed_copies) b = Operand{yt + c0, plan.ld_yt, false};   // [d][K = cols] K-major
                    t_tag = TAG_DX;
                    rc = launch_gemm(EPI_OUT, a, b, nr, dn, nc, pick_contraction_bn(nr, dn, overlap, transposed_copies), p, sx);
                    if (rc) return rc;
                    if (overlap) MECLIP_CUDA(cudaEventRecord(side->dx[gb], sx));
                }
            }
        }
    }
    if (overlap) {   // join: everything the side streams did is ordered before the caller's next work
        if (want_dx) {
            MECLIP_CUDA(cudaEventRecord(side->join_x, sx));
            MECLIP_CUDA(cudaStreamWaitEvent(s0, side->join_x, 0));
        }
        if (want_dy) {
            MECLIP_CUDA(cudaEventRecord(side->join_y, sy));
            MECLIP_CUDA(cudaStreamWaitEvent(s0, side->join_y, 0));
        }
    }
    return MECLIP_OK;
}

}  // namespace meclip

extern "C" {

int meclip_grad(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                int64_t ldy, float temperature, int64_t row_off, int64_t col_off, const float* row_sum,
                const float* col_sum, const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx,
                void* dy, int dy_mode, int64_t lddy, void* workspace, size_t workspace_bytes, int* status,
                void* stream) {
    const DeviceScalars ds = take_scalars();
    return grad_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                     grad_out, grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, workspace, workspace_bytes, status,
                     (cudaStream_t)stream, overlap_allowed(), transposes_allowed(), nullptr, 0.f, 0.f, 0, false, ds);
}

int meclip_grad_t(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                  int64_t ldy, float temperature, int64_t row_off, int64_t col_off, const float* row_sum,
                  const float* col_sum, const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx,
                  void* dy, int dy_mode, int64_t lddy, float* sum_g_s, void* workspace, size_t workspace_bytes,
                  int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (sum_g_s == nullptr) return fail(MECLIP_EINVAL, "grad_t: sum_g_s is null");
    return grad_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                     grad_out, grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, workspace, workspace_bytes, status,
                     (cudaStream_t)stream, overlap_allowed(), transposes_allowed(), sum_g_s, 0.f, 0.f, 0, false, ds);
}

int meclip_grad_tf32(int kind, const void* x_bf16, const void* y_bf16, const float* x_f32, int64_t ldxf,
                     const float* y_f32, int64_t ldyf, int64_t rows, int64_t cols, int64_t d, int64_t ldx, int64_t ldy,
                     float temperature, int64_t row_off, int64_t col_off, const float* row_sum, const float* col_sum,
                     const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy, int dy_mode,
                     int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (x_f32 == nullptr || y_f32 == nullptr) return fail(MECLIP_EINVAL, "grad_tf32: fp32 operands are null");
    return grad_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                     grad_out, grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, workspace, workspace_bytes, status,
                     (cudaStream_t)stream, overlap_allowed(), transposes_allowed(), nullptr, 0.f, 0.f, 0, false, ds, true,
                     x_f32, ldxf, y_f32, ldyf);
}

// ---- LiT forward that already holds the gradient's contraction ------------------------------------
int meclip_lit_extend(void* y_bf16, int64_t rows, int64_t d, int64_t ldy, void* stream) {
    if (y_bf16 == nullptr || rows < 1 || d < 8 || d % 8 != 0 || ldy < d + 8 || ldy % 8 != 0 || !aligned16(y_bf16))
        return fail(MECLIP_EINVAL, "lit_extend: need a 16-byte aligned matrix with d a multiple of 8 and ld >= d + 8");
    ScopedTiming timing((cudaStream_t)stream, TAG_ROW, (double)rows * 16.0);
    ones_column_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)y_bf16, rows, d, ldy);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_lit_fused_forward(const void* x_bf16, const void* y_ext_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                             int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* u, int u_mode,
                             int64_t ldu, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    DeviceScalars ds = take_scalars();
    ds.g_rule = 0;            // the panel holds E itself here: no gradient scale to adjust
    if (u == nullptr) return fail(MECLIP_EINVAL, "lit_fused_forward: u is null");
    if (u_mode != MECLIP_STORE_F32 && u_mode != MECLIP_ACCUM_F32) return fail(MECLIP_EINVAL, "lit_fused_forward: u is fp32");
    return grad_impl(MECLIP_LIT, x_bf16, y_ext_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, nullptr, nullptr,
                     nullptr, 1.f, u, u_mode, ldu, nullptr, 0, 0, workspace, workspace_bytes, status, (cudaStream_t)stream,
                     overlap_allowed(), transposes_allowed(), nullptr, 0.f, 0.f, 8, true, ds);
}

int meclip_lit_fused_stats(const void* x_bf16, int64_t ldx, const void* y_ext_bf16, int64_t ldy, const float* u, int64_t ldu,
                           int64_t rows, int64_t d, float* row_sum, float* diag_s, void* stream) {
    if (x_bf16 == nullptr || y_ext_bf16 == nullptr || u == nullptr || row_sum == nullptr || diag_s == nullptr)
        return fail(MECLIP_EINVAL, "lit_fused_stats: null pointer");
    if (rows < 1 || d < 8 || d % 8 != 0 || ldx < d || ldy < d + 8 || ldu < d + 8 || ldx % 8 != 0 || ldy % 8 != 0 ||
        !aligned16(x_bf16) || !aligned16(y_ext_bf16))
        return fail(MECLIP_EINVAL, "lit_fused_stats: bad shape or alignment");
    const int wpb = ROW_KERNEL_THREADS / 32;
    ScopedTiming timing((cudaStream_t)stream, TAG_ROW, (double)rows * ((double)d * 4 + 12));
    lit_fused_stats_kernel<<<(unsigned)((rows + wpb - 1) / wpb), ROW_KERNEL_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x_bf16, ldx, (const __nv_bfloat16*)y_ext_bf16, ldy, u, ldu, rows, (int)d, row_sum, diag_s);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_lit_fused_backward(const float* u, int64_t ldu, const void* y_ext_bf16, int64_t ldy, const float* row_sum,
                              const float* grad_out, float grad_scale, int64_t rows, int64_t d, void* dx, int dx_dtype,
                              int64_t lddx, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (u == nullptr || y_ext_bf16 == nullptr || row_sum == nullptr || dx == nullptr)
        return fail(MECLIP_EINVAL, "lit_fused_backward: null pointer");
    if (rows < 1 || d < 1 || ldu < d || ldy < d || lddx < d || ldu % 4 != 0 || ldy % 8 != 0 || !aligned16(u) || !aligned16(y_ext_bf16))
        return fail(MECLIP_EINVAL, "lit_fused_backward: bad shape or alignment");
    const int oelt = dx_dtype == MECLIP_F32 ? 4 : 2;
    const int vec_out = (d % 8 == 0) && aligned16(dx) && ((lddx * oelt) % 16 == 0);
    const int wpb = ROW_KERNEL_THREADS / 32;
    const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16* y = (const __nv_bfloat16*)y_ext_bf16;
    ScopedTiming timing(s, TAG_NORM_BWD, (double)rows * (double)d * (6.0 + oelt));
    if (dx_dtype == MECLIP_F32)
        lit_fused_bwd_kernel<float><<<grid, ROW_KERNEL_THREADS, 0, s>>>(u, ldu, y, ldy, row_sum, grad_out, grad_scale, ds.t, ds.g_rule, rows, (int)d, vec_out, (float*)dx, lddx);
    else if (dx_dtype == MECLIP_BF16)
        lit_fused_bwd_kernel<__nv_bfloat16><<<grid, ROW_KERNEL_THREADS, 0, s>>>(u, ldu, y, ldy, row_sum, grad_out, grad_scale, ds.t, ds.g_rule, rows, (int)d, vec_out, (__nv_bfloat16*)dx, lddx);
    else if (dx_dtype == MECLIP_F16)
        lit_fused_bwd_kernel<__half><<<grid, ROW_KERNEL_THREADS, 0, s>>>(u, ldu, y, ldy, row_sum, grad_out, grad_scale, ds.t, ds.g_rule, rows, (int)d, vec_out, (__half*)dx, lddx);
    else
        return fail(MECLIP_EINVAL, "lit_fused_backward: bad output dtype %d", dx_dtype);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

// ---- sigmoid (SigLIP) loss on the same tile engine -------------------------------------------------
int meclip_siglip_sum(const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                      int64_t ldy, float logit_scale, float logit_bias, int64_t row_off, int64_t col_off, float* row_sum,
                      float* diag_s, unsigned int* tile_counter, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (x_bf16 == nullptr || y_bf16 == nullptr || row_sum == nullptr || diag_s == nullptr)
        return fail(MECLIP_EINVAL, "siglip_sum: null pointer");
    if (rows < 1 || cols < 1 || d < 8 || d % 8 != 0 || ldx < d || ldy < d)
        return fail(MECLIP_EINVAL, "siglip_sum: need rows, cols >= 1, d a multiple of 8, ld >= d");
    int rc = check_device();
    if (rc) return rc;
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.sigmoid = 1;
    p.fmul = logit_scale * 1.4426950408889634f;
    p.fadd = logit_bias * 1.4426950408889634f;
    p.t_dev = ds.t;
    p.b_dev = ds.b;
    p.diag_shift = (long long)row_off - (long long)col_off;
    p.row_sum = row_sum;
    p.col_sum = nullptr;
    p.diag = diag_s;
    p.tile_counter = tile_counter;
    p.status = status;
    Operand a{x_bf16, ldx, false}, b{y_bf16, ldy, false};
    t_tag = TAG_SUMS;
    return launch_gemm(EPI_SUMS, a, b, rows, cols, d, pick_bn(cols), p, (cudaStream_t)stream);
}

int meclip_siglip_loss_finalize(const float* row_sum, const float* diag_s, int64_t n, float logit_scale, float logit_bias,
                                float scale, int accumulate, float* loss_out, void* stream) {
    if (row_sum == nullptr || diag_s == nullptr || loss_out == nullptr || n < 1)
        return fail(MECLIP_EINVAL, "siglip_loss_finalize: bad argument");
    ScopedTiming timing((cudaStream_t)stream, TAG_ROW, 0.0);
    siglip_finalize_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(row_sum, diag_s, n, logit_scale, logit_bias, scale,
                                                                 accumulate, loss_out);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_siglip_grad(const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                       int64_t ldy, float logit_scale, float logit_bias, int64_t row_off, int64_t col_off,
                       const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy,
                       int dy_mode, int64_t lddy, float* sums, void* workspace, size_t workspace_bytes, int* status,
                       void* stream) {
    const DeviceScalars ds = take_scalars();
    return grad_impl(MECLIP_SIGLIP, x_bf16, y_bf16, rows, cols, d, ldx, ldy, 1.f, row_off, col_off, nullptr, nullptr,
                     grad_out, grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, workspace, workspace_bytes, status,
                     (cudaStream_t)stream, overlap_allowed(), transposes_allowed(), sums, logit_scale, logit_bias, 0, false,
                     ds);
}

int meclip_loss_forward(int kind, const void* x_bf16, const void* y_bf16, int64_t batch, int64_t d, int64_t ldx,
                        int64_t ldy, float temperature, float* row_sum, float* col_sum, float* diag_s, float* loss_out,
                        unsigned int* tile_counter, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    NvtxRange range("meclip_loss_forward");
    if (batch < 1 || row_sum == nullptr || diag_s == nullptr || loss_out == nullptr)
        return fail(MECLIP_EINVAL, "loss_forward: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    MECLIP_CUDA(cudaMemsetAsync(row_sum, 0, (size_t)batch * sizeof(float), s));
    if (kind == MECLIP_CLIP && col_sum != nullptr) MECLIP_CUDA(cudaMemsetAsync(col_sum, 0, (size_t)batch * sizeof(float), s));
    MECLIP_CUDA(cudaMemsetAsync(diag_s, 0, (size_t)batch * sizeof(float), s));
    if (tile_counter != nullptr) MECLIP_CUDA(cudaMemsetAsync(tile_counter, 0, sizeof(unsigned int), s));
    int rc = sum_exp_impl(kind, x_bf16, y_bf16, batch, batch, d, ldx, ldy, temperature, 0, 0, row_sum, col_sum, diag_s,
                          tile_counter, status, stream, ds);
    if (rc) return rc;
    return loss_finalize_impl(kind, row_sum, col_sum, diag_s, batch, temperature, 1.0f / (float)batch, 0, loss_out,
                              stream, ds);
}

int meclip_loss_backward(int kind, const void* x_bf16, const void* y_bf16, int64_t batch, int64_t d, int64_t ldx,
                         int64_t ldy, float temperature, const float* row_sum, const float* col_sum,
                         const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy,
                         int dy_mode, int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    return meclip_grad(kind, x_bf16, y_bf16, batch, batch, d, ldx, ldy, temperature, 0, 0, row_sum, col_sum, grad_out,
                       grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, workspace, workspace_bytes, status, stream);
}

// ------------------------------------------------------------------------------------
// whole-step entry points for small batches (the step is host-bound there)
// ------------------------------------------------------------------------------------
}  // extern "C"

namespace meclip {
struct StepLayout {
    long long dp;
    size_t x_hat, y_hat, inv_x, inv_y, row_sum, col_sum, diag, counter, stats_bytes, total;
};
static StepLayout step_layout(int64_t b, int64_t d) {
    StepLayout l;
    l.dp = (long long)round_up((size_t)d, 8);
    const size_t op = round_up((size_t)b * l.dp * 2, 256), vec = round_up((size_t)b * 4, 256);
    l.x_hat = 0;
    l.y_hat = op;
    l.inv_x = 2 * op;
    l.inv_y = l.inv_x + vec;
    l.row_sum = l.inv_y + vec;            // row_sum | col_sum | diag | counter are cleared by ONE memset
    l.col_sum = l.row_sum + vec;
    l.diag = l.col_sum + vec;
    l.counter = l.diag + vec;
    l.stats_bytes = 3 * vec + 256;
    l.total = l.counter + 256;
    return l;
}
}  // namespace meclip

extern "C" {

size_t meclip_step_saved_bytes(int64_t batch, int64_t d) {
    if (batch < 1 || d < 1) return 0;
    return step_layout(batch, d).total;
}

size_t meclip_step_workspace_bytes(int64_t batch, int64_t d) {
    if (batch < 1 || d < 1) return 0;
    const StepLayout l = step_layout(batch, d);
    return 2 * round_up((size_t)batch * l.dp * 4, 256) + plan_grad(batch, batch, l.dp, false).total() + 256;
}

int meclip_step_forward(int kind, const void* x, const void* y, int in_dtype, int64_t batch, int64_t d, int64_t ldx,
                        int64_t ldy, int normalize, float temperature, void* saved, size_t saved_bytes, float* loss_out,
                        int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    NvtxRange range("meclip_step_forward");
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT) return fail(MECLIP_EINVAL, "step_forward: bad kind %d", kind);
    if (x == nullptr || y == nullptr || saved == nullptr || loss_out == nullptr) return fail(MECLIP_EINVAL, "step_forward: null pointer");
    if (batch < 1 || d < 1 || ldx < d || ldy < d) return fail(MECLIP_EINVAL, "step_forward: need batch, d >= 1 and ld >= d");
    if ((reinterpret_cast<uintptr_t>(saved) & 255u) != 0) return fail(MECLIP_EINVAL, "step_forward: saved must be 256-byte aligned");
    const StepLayout l = step_layout(batch, d);
    if (saved_bytes < l.total) return fail(MECLIP_ENOSPC, "step_forward: saved buffer %zu < %zu bytes", saved_bytes, l.total);
    const int elt = in_dtype == MECLIP_F32 ? 4 : 2;
    if (in_dtype != MECLIP_F32 && in_dtype != MECLIP_BF16 && in_dtype != MECLIP_F16) return fail(MECLIP_EINVAL, "step_forward: bad dtype %d", in_dtype);
    uint8_t* sv = reinterpret_cast<uint8_t*>(saved);
    __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(sv + l.x_hat);
    __nv_bfloat16* yh = reinterpret_cast<__nv_bfloat16*>(sv + l.y_hat);
    float* inv_x = reinterpret_cast<float*>(sv + l.inv_x);
    float* inv_y = reinterpret_cast<float*>(sv + l.inv_y);
    cudaStream_t s = (cudaStream_t)stream;
    {   // (1) both inputs: normalise (or convert) to bf16 operands, one launch
        const int vec0 = (d % 8 == 0) && aligned16(x) && ((ldx * elt) % 16 == 0);
        const int vec1 = (d % 8 == 0) && aligned16(y) && ((ldy * elt) % 16 == 0);
        const int wpb = ROW_KERNEL_THREADS / 32;
        dim3 grid((unsigned)((batch + wpb - 1) / wpb), 2);
        ScopedTiming timing(s, TAG_NORM_FWD, 2.0 * (double)batch * ((double)d * elt + (double)l.dp * 2 + (normalize ? 4 : 0)));
        if (in_dtype == MECLIP_F32)
            normalize_fwd_pair_kernel<float><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const float*)x, ldx, vec0, xh, inv_x, (const float*)y, ldy, vec1, yh, inv_y, batch, (int)d, (int)l.dp, normalize, l.dp);
        else if (in_dtype == MECLIP_BF16)
            normalize_fwd_pair_kernel<__nv_bfloat16><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const __nv_bfloat16*)x, ldx, vec0, xh, inv_x, (const __nv_bfloat16*)y, ldy, vec1, yh, inv_y, batch, (int)d, (int)l.dp, normalize, l.dp);
        else
            normalize_fwd_pair_kernel<__half><<<grid, ROW_KERNEL_THREADS, 0, s>>>((const __half*)x, ldx, vec0, xh, inv_x, (const __half*)y, ldy, vec1, yh, inv_y, batch, (int)d, (int)l.dp, normalize, l.dp);
        MECLIP_CUDA(cudaGetLastError());
    }
    // (2) sums, diagonal and the tile counter in one clear
    MECLIP_CUDA(cudaMemsetAsync(sv + l.row_sum, 0, l.stats_bytes, s));
    // (3) tile pass, (4) loss
    float* row_sum = reinterpret_cast<float*>(sv + l.row_sum);
    float* col_sum = kind == MECLIP_CLIP ? reinterpret_cast<float*>(sv + l.col_sum) : nullptr;
    float* diag = reinterpret_cast<float*>(sv + l.diag);
    int rc = sum_exp_impl(kind, xh, yh, batch, batch, l.dp, l.dp, l.dp, temperature, 0, 0, row_sum, col_sum, diag,
                          reinterpret_cast<unsigned int*>(sv + l.counter), status, stream, ds);
    if (rc) return rc;
    return loss_finalize_impl(kind, row_sum, col_sum, diag, batch, temperature, 1.0f / (float)batch, 0, loss_out, stream, ds);
}

int meclip_step_backward(int kind, const void* saved, size_t saved_bytes, int64_t batch, int64_t d, int normalize,
                         float temperature, const float* grad_out, float grad_scale, void* dx, void* dy, int out_dtype,
                         int64_t lddx, int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    NvtxRange range("meclip_step_backward");
    if (kind == MECLIP_LIT) dy = nullptr;       // the second argument of LiT gets no gradient (lit_loss.py:247)
    if (saved == nullptr || workspace == nullptr || (dx == nullptr && dy == nullptr)) return fail(MECLIP_EINVAL, "step_backward: null pointer");
    if (batch < 1 || d < 1 || (dx != nullptr && lddx < d) || (dy != nullptr && lddy < d)) return fail(MECLIP_EINVAL, "step_backward: bad shape");
    if (out_dtype != MECLIP_F32 && out_dtype != MECLIP_BF16 && out_dtype != MECLIP_F16) return fail(MECLIP_EINVAL, "step_backward: bad dtype %d", out_dtype);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(MECLIP_EINVAL, "step_backward: workspace must be 256-byte aligned");
    const StepLayout l = step_layout(batch, d);
    if (saved_bytes < l.total) return fail(MECLIP_ENOSPC, "step_backward: saved buffer %zu < %zu bytes", saved_bytes, l.total);
    if (workspace_bytes < meclip_step_workspace_bytes(batch, d)) return fail(MECLIP_ENOSPC, "step_backward: workspace too small");
    const uint8_t* sv = reinterpret_cast<const uint8_t*>(saved);
    const __nv_bfloat16* xh = reinterpret_cast<const __nv_bfloat16*>(sv + l.x_hat);
    const __nv_bfloat16* yh = reinterpret_cast<const __nv_bfloat16*>(sv + l.y_hat);
    const float* row_sum = reinterpret_cast<const float*>(sv + l.row_sum);
    const float* col_sum = kind == MECLIP_CLIP ? reinterpret_cast<const float*>(sv + l.col_sum) : nullptr;
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const size_t g32 = round_up((size_t)batch * l.dp * 4, 256);
    float* dx32 = reinterpret_cast<float*>(ws);
    float* dy32 = reinterpret_cast<float*>(ws + g32);
    uint8_t* gws = ws + 2 * g32;
    const size_t gws_bytes = workspace_bytes - 2 * g32;
    const int oelt = out_dtype == MECLIP_F32 ? 4 : 2;
    // the contractions write the outputs themselves when no Jacobian follows and they can (dtype, 16-byte rows)
    const bool direct = !normalize && out_dtype != MECLIP_F16 && d % 8 == 0 &&
                        (dx == nullptr || (aligned16(dx) && lddx % 8 == 0)) && (dy == nullptr || (aligned16(dy) && lddy % 8 == 0));
    const int mode = direct ? (out_dtype == MECLIP_BF16 ? MECLIP_STORE_BF16 : MECLIP_STORE_F32) : MECLIP_STORE_F32;
    // one stream, no transposed operand copies: at these sizes every extra launch costs more than it saves
    int rc = grad_impl(kind, xh, yh, batch, batch, l.dp, l.dp, l.dp, temperature, 0, 0, row_sum, col_sum, grad_out, grad_scale,
                       dx == nullptr ? nullptr : (direct ? dx : (void*)dx32), mode, direct ? lddx : l.dp,
                       dy == nullptr ? nullptr : (direct ? dy : (void*)dy32), mode, direct ? lddy : l.dp, gws, gws_bytes, status,
                       (cudaStream_t)stream, false, false, nullptr, 0.f, 0.f, 0, false, ds);
    if (rc || direct) return rc;
    // Jacobian of the normalisation (or the plain conversion) for both gradients in one launch
    cudaStream_t s = (cudaStream_t)stream;
    const float* inv_x = normalize ? reinterpret_cast<const float*>(sv + l.inv_x) : nullptr;
    const float* inv_y = normalize ? reinterpret_cast<const float*>(sv + l.inv_y) : nullptr;
    const int wpb = ROW_KERNEL_THREADS / 32;
    const bool both = dx != nullptr && dy != nullptr;
    dim3 grid((unsigned)((batch + wpb - 1) / wpb), both ? 2 : 1);
    // with one output only, it takes slot 0 of the pair kernel
    const float* g0 = dx != nullptr ? dx32 : dy32;
    const __nv_bfloat16* h0 = dx != nullptr ? xh : yh;
    const float* i0 = dx != nullptr ? inv_x : inv_y;
    void* o0 = dx != nullptr ? dx : dy;
    const int64_t ld0 = dx != nullptr ? lddx : lddy;
    const int v0 = (d % 8 == 0) && aligned16(o0) && ((ld0 * oelt) % 16 == 0);
    const int v1 = both && (d % 8 == 0) && aligned16(dy) && ((lddy * oelt) % 16 == 0);
    ScopedTiming timing(s, TAG_NORM_BWD, (both ? 2.0 : 1.0) * (double)batch * ((double)l.dp * 6 + (double)d * oelt + 4));
    if (out_dtype == MECLIP_F32)
        normalize_bwd_pair_kernel<float><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g0, h0, i0, v0, (float*)o0, ld0, dy32, yh, inv_y, v1, (float*)dy, lddy, l.dp, l.dp, batch, (int)d);
    else if (out_dtype == MECLIP_BF16)
        normalize_bwd_pair_kernel<__nv_bfloat16><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g0, h0, i0, v0, (__nv_bfloat16*)o0, ld0, dy32, yh, inv_y, v1, (__nv_bfloat16*)dy, lddy, l.dp, l.dp, batch, (int)d);
    else
        normalize_bwd_pair_kernel<__half><<<grid, ROW_KERNEL_THREADS, 0, s>>>(g0, h0, i0, v0, (__half*)o0, ld0, dy32, yh, inv_y, v1, (__half*)dy, lddy, l.dp, l.dp, batch, (int)d);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

// ------------------------------------------------------------------------------------
// backward without a caller-provided workspace
// ------------------------------------------------------------------------------------
// The coefficient panel of meclip_grad_static lives here instead of in caller memory.
// 4096 x 4096 bf16 = 32 MiB (+ 4 KiB for tile counters), resident on every GPU that loads this library until the
// process exits.  In host code the name below is only a handle for the symbol, not a
// device address: static_scratch_ptr() asks the runtime for the real address once per device.
static constexpr long long STATIC_MAX_ROWS = 4096;
static constexpr long long STATIC_MAX_COLS = 4096;
static constexpr size_t STATIC_SCRATCH_BYTES = (size_t)STATIC_MAX_ROWS * STATIC_MAX_COLS * 2 + 4096;  // panel + tile counters
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[64] = {nullptr};

static int static_scratch_ptr(void** out) {
    int dev = 0;
    MECLIP_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MECLIP_EUNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        MECLIP_CUDA(cudaSetDevice(dev));   // the symbol is looked up in the current device's copy of the module
        MECLIP_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255u) != 0)
            return fail(MECLIP_ECUDA, "static scratch: bad symbol address %p", ptr);
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return MECLIP_OK;
}

int meclip_grad_static(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                       int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off,
                       const float* row_sum, const float* col_sum, const float* grad_out, float grad_scale, void* dx,
                       int dx_mode, int64_t lddx, void* dy, int dy_mode, int64_t lddy, int* status, void* stream) {
    const DeviceScalars ds = take_scalars();
    if (rows < 1 || cols < 1) return fail(MECLIP_EINVAL, "grad_static: rows and cols must be >= 1");
    if (rows > STATIC_MAX_ROWS || cols > STATIC_MAX_COLS)
        return fail(MECLIP_ENOSPC,
                    "grad_static: block %lld x %lld exceeds the built-in scratch (at most %lld x %lld); "
                    "use meclip_grad with a caller workspace",
                    (long long)rows, (long long)cols, STATIC_MAX_ROWS, STATIC_MAX_COLS);
    void* scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    // The scratch keeps the previous call's contents.  The panel needs no clearing: every element
    // that is read was written by this call first and the tile loads are bounded to the rows x cols
    // written.  The tile counters behind it must start at zero and are cleared on the stream first.
    // All launches stay on the caller's stream; no stream, event or memory is created, and the
    // contractions read X and Y as they are (no transposed copies, which would need more scratch).
    // The plan is made from the built-in constants: the test hook and the environment switches that change the
    // blocking of meclip_grad do not apply here, so every block within the limit fits the scratch as one panel.
    return grad_impl(kind, x_bf16, y_bf16, rows, cols, d, ldx, ldy, temperature, row_off, col_off, row_sum, col_sum,
                     grad_out, grad_scale, dx, dx_mode, lddx, dy, dy_mode, lddy, scratch, STATIC_SCRATCH_BYTES,
                     status, (cudaStream_t)stream, false, false, nullptr, 0.f, 0.f, 0, false, ds, false);
}

// ------------------------------------------------------------------------------------
// peer memory of another process on the same node (ring: shards fetched by the copy engines)
// ------------------------------------------------------------------------------------
int meclip_ipc_export(const void* ptr, void* handle_out, uint64_t* offset_out) {
    if (ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return fail(MECLIP_EINVAL, "ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == MECLIP_IPC_HANDLE_BYTES, "handle size");
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range_fn = []() -> RangeFn {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        return q == cudaDriverEntryPointSuccess ? reinterpret_cast<RangeFn>(f) : nullptr;
    }();
    if (range_fn == nullptr) return fail(MECLIP_EUNSUPPORTED, "ipc_export: cuMemGetAddressRange not available");
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range_fn(&base, &size, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS)
        return fail(MECLIP_ECUDA, "ipc_export: %p is not inside a device allocation", ptr);
    cudaIpcMemHandle_t h;
    MECLIP_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base)));
    std::memcpy(handle_out, &h, sizeof(h));
    *offset_out = (uint64_t)((uintptr_t)ptr - (uintptr_t)base);
    return MECLIP_OK;
}

int meclip_ipc_open(const void* handle, void** base_out) {
    if (handle == nullptr || base_out == nullptr) return fail(MECLIP_EINVAL, "ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    MECLIP_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *base_out = base;
    return MECLIP_OK;
}

int meclip_ipc_close(void* base) {
    if (base == nullptr) return fail(MECLIP_EINVAL, "ipc_close: null pointer");
    MECLIP_CUDA(cudaIpcCloseMemHandle(base));
    return MECLIP_OK;
}

int meclip_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
    if (dst == nullptr || src == nullptr) return fail(MECLIP_EINVAL, "copy_async: null pointer");
    if (bytes == 0) return MECLIP_OK;
    MECLIP_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return MECLIP_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------
// the ring of one rank, queued in one call: tile kernels on the compute stream, shard
// fetches and partial-gradient pushes on the copy stream (copy engines, peer memory)
// ------------------------------------------------------------------------------------
struct RingEvents {
    bool ready = false;
    cudaEvent_t fetched[2] = {nullptr, nullptr};     // shard of step s landed in recv[s & 1]
    cudaEvent_t kernels[2] = {nullptr, nullptr};     // kernels of step s are done (recv[s & 1], part[s & 1] free)
    cudaEvent_t pushed[2] = {nullptr, nullptr};      // partial of step s left part[s & 1]
    std::mutex mutex;
};
static RingEvents g_ring[64];
static std::mutex g_ring_init_mutex;

static int get_ring_events(RingEvents** out) {
    int dev = 0;
    MECLIP_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MECLIP_EUNSUPPORTED, "device index %d out of range", dev);
    RingEvents& re = g_ring[dev];
    std::lock_guard<std::mutex> lock(g_ring_init_mutex);
    if (!re.ready) {
        cudaEvent_t* evs[6] = {&re.fetched[0], &re.fetched[1], &re.kernels[0], &re.kernels[1], &re.pushed[0], &re.pushed[1]};
        for (auto e : evs) MECLIP_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        re.ready = true;
    }
    *out = &re;
    return MECLIP_OK;
}

static int ring_check(const meclip_ring_desc* r, const char* who) {
    if (r == nullptr) return fail(MECLIP_EINVAL, "%s: ring descriptor is null", who);
    if (r->nranks < 1 || r->rank < 0 || r->rank >= r->nranks)
        return fail(MECLIP_EINVAL, "%s: rank %d of %d", who, r->rank, r->nranks);
    if (r->rows < 1 || r->d < 8 || r->d % 8 != 0 || r->ldx < r->d || r->ldy < r->d)
        return fail(MECLIP_EINVAL, "%s: rows=%lld d=%lld ldx=%lld ldy=%lld", who, (long long)r->rows, (long long)r->d,
                    (long long)r->ldx, (long long)r->ldy);
    if (r->shards == nullptr) return fail(MECLIP_EINVAL, "%s: shards is null", who);
    for (int p = 0; p < r->nranks; ++p)
        if (r->shards[p] == nullptr || !aligned16(r->shards[p])) return fail(MECLIP_EINVAL, "%s: shards[%d] is null or not 16-byte aligned", who, p);
    if (r->nranks > 1) {
        if (r->recv[1] == nullptr || (r->nranks > 2 && r->recv[0] == nullptr)) return fail(MECLIP_EINVAL, "%s: receive buffer is null", who);
        if (r->compute_stream == r->copy_stream) return fail(MECLIP_EINVAL, "%s: compute and copy stream must differ", who);
    }
    return MECLIP_OK;
}

// The operand of ring step `step`: the own shard at step 0, else the receive buffer the fetch of that step went to.
// Queues the fetch of step + 1 first, so that it runs under this step's kernels.
static int ring_operand(const meclip_ring_desc* r, RingEvents* re, int step, const void** y_out) {
    cudaStream_t compute = (cudaStream_t)r->compute_stream, copy = (cudaStream_t)r->copy_stream;
    const size_t shard_bytes = (size_t)r->rows * (size_t)r->ldy * 2;
    if (step + 1 < r->nranks) {
        const int slot = (step + 1) & 1;
        if (step >= 1) MECLIP_CUDA(cudaStreamWaitEvent(copy, re->kernels[slot], 0));   // step - 1 read this buffer
        MECLIP_CUDA(cudaMemcpyAsync(r->recv[slot], r->shards[(r->rank + step + 1) % r->nranks], shard_bytes,
                                    cudaMemcpyDeviceToDevice, copy));
        MECLIP_CUDA(cudaEventRecord(re->fetched[slot], copy));
    }
    if (step == 0) {
        *y_out = r->shards[r->rank];
    } else {
        MECLIP_CUDA(cudaStreamWaitEvent(compute, re->fetched[step & 1], 0));
        *y_out = r->recv[step & 1];
    }
    return MECLIP_OK;
}

extern "C" {

int meclip_ring_sum_exp(const meclip_ring_desc* r, int kind, const void* x_bf16, float temperature, float* row_sum,
                        float* col_part, float* diag_s, unsigned int* tile_counters, int* status) {
    const DeviceScalars ds = take_scalars();
    int rc = ring_check(r, "ring_sum_exp");
    if (rc != MECLIP_OK) return rc;
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT) return fail(MECLIP_EINVAL, "ring_sum_exp: kind %d", kind);
    if (x_bf16 == nullptr || row_sum == nullptr || diag_s == nullptr || tile_counters == nullptr ||
        (kind == MECLIP_CLIP && col_part == nullptr))
        return fail(MECLIP_EINVAL, "ring_sum_exp: null pointer");
    RingEvents* re = nullptr;
    rc = get_ring_events(&re);
    if (rc != MECLIP_OK) return rc;
    std::lock_guard<std::mutex> lock(re->mutex);
    NvtxRange range("meclip_ring_sum_exp");
    cudaStream_t compute = (cudaStream_t)r->compute_stream;
    const int64_t b = r->rows;
    MECLIP_CUDA(cudaMemsetAsync(row_sum, 0, (size_t)b * 4, compute));
    MECLIP_CUDA(cudaMemsetAsync(diag_s, 0, (size_t)b * 4, compute));
    MECLIP_CUDA(cudaMemsetAsync(tile_counters, 0, (size_t)r->nranks * 4, compute));
    if (kind == MECLIP_CLIP) MECLIP_CUDA(cudaMemsetAsync(col_part, 0, (size_t)r->nranks * (size_t)b * 4, compute));
    for (int step = 0; step < r->nranks; ++step) {
        const int shard = (r->rank + step) % r->nranks;
        const void* y = nullptr;
        rc = ring_operand(r, re, step, &y);
        if (rc != MECLIP_OK) return rc;
        rc = sum_exp_impl(kind, x_bf16, y, b, b, r->d, r->ldx, r->ldy, temperature, (int64_t)r->rank * b, (int64_t)shard * b,
                          row_sum, kind == MECLIP_CLIP ? col_part + (size_t)shard * b : nullptr, diag_s,
                          tile_counters + step, status, r->compute_stream, ds);
        if (rc != MECLIP_OK) return rc;
        MECLIP_CUDA(cudaEventRecord(re->kernels[step & 1], compute));
    }
    return MECLIP_OK;
}

int meclip_ring_grad(const meclip_ring_desc* r, int kind, const void* x_bf16, float temperature, const float* row_sum,
                     const float* col_sum_all, const float* grad_out, float grad_scale, float* dx_acc, int64_t lddx,
                     float* dy_own, float* part0, float* part1, void* const* inbox, void* workspace,
                     size_t workspace_bytes, int* status) {
    const DeviceScalars ds = take_scalars();
    int rc = ring_check(r, "ring_grad");
    if (rc != MECLIP_OK) return rc;
    if (kind != MECLIP_CLIP && kind != MECLIP_LIT) return fail(MECLIP_EINVAL, "ring_grad: kind %d", kind);
    const bool want_dy = kind == MECLIP_CLIP;
    const bool exchange = want_dy && r->nranks > 1;
    if (x_bf16 == nullptr || row_sum == nullptr || dx_acc == nullptr || workspace == nullptr || lddx < r->d ||
        (want_dy && (col_sum_all == nullptr || dy_own == nullptr)))
        return fail(MECLIP_EINVAL, "ring_grad: null pointer or lddx < d");
    if (exchange) {
        if (part1 == nullptr || (r->nranks > 2 && part0 == nullptr) || inbox == nullptr)
            return fail(MECLIP_EINVAL, "ring_grad: partial buffers or inbox table are null");
        for (int p = 0; p < r->nranks; ++p)
            if (p != r->rank && inbox[p] == nullptr) return fail(MECLIP_EINVAL, "ring_grad: inbox[%d] is null", p);
    }
    RingEvents* re = nullptr;
    rc = get_ring_events(&re);
    if (rc != MECLIP_OK) return rc;
    std::lock_guard<std::mutex> lock(re->mutex);
    NvtxRange range("meclip_ring_grad");
    cudaStream_t compute = (cudaStream_t)r->compute_stream, copy = (cudaStream_t)r->copy_stream;
    const int64_t b = r->rows;
    const size_t slot_bytes = (size_t)b * (size_t)r->d * 4;
    float* part[2] = {part0, part1};
    MECLIP_CUDA(cudaMemsetAsync(dx_acc, 0, (size_t)b * (size_t)lddx * 4, compute));
    for (int step = 0; step < r->nranks; ++step) {
        const int shard = (r->rank + step) % r->nranks;
        const void* y = nullptr;
        rc = ring_operand(r, re, step, &y);
        if (rc != MECLIP_OK) return rc;
        float* out = nullptr;
        if (want_dy) {
            out = step == 0 ? dy_own : part[step & 1];
            if (step >= 3) MECLIP_CUDA(cudaStreamWaitEvent(compute, re->pushed[step & 1], 0));   // push of step - 2
        }
        rc = grad_impl(kind, x_bf16, y, b, b, r->d, r->ldx, r->ldy, temperature, (int64_t)r->rank * b, (int64_t)shard * b,
                       row_sum, want_dy ? col_sum_all + (size_t)shard * b : nullptr, grad_out, grad_scale, dx_acc,
                       MECLIP_ACCUM_F32, lddx, out, MECLIP_STORE_F32, r->d, workspace, workspace_bytes, status, compute,
                       overlap_allowed(), transposes_allowed(), nullptr, 0.f, 0.f, 0, false, ds);
        if (rc != MECLIP_OK) return rc;
        MECLIP_CUDA(cudaEventRecord(re->kernels[step & 1], compute));
        if (exchange && step >= 1) {
            char* dst = static_cast<char*>(inbox[shard]) + (size_t)(step - 1) * slot_bytes;
            MECLIP_CUDA(cudaStreamWaitEvent(copy, re->kernels[step & 1], 0));
            MECLIP_CUDA(cudaMemcpyAsync(dst, out, slot_bytes, cudaMemcpyDeviceToDevice, copy));
            MECLIP_CUDA(cudaEventRecord(re->pushed[step & 1], copy));
        }
    }
    return MECLIP_OK;
}

int meclip_debug_wait_probe(uint64_t limit_ns, int* status, void* stream) {
    if (status == nullptr) return fail(MECLIP_EINVAL, "wait_probe: status is null");
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail(MECLIP_EINVAL, "wait_probe: limit must be in (0, 100 ms]");
    ScopedTiming timing((cudaStream_t)stream, TAG_ROW, 0.0);
    wait_probe_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, status);
    MECLIP_CUDA(cudaGetLastError());
    return MECLIP_OK;
}

int meclip_debug_gemm(const void* a_bf16, int64_t lda, int a_mn_major, const void* b_bf16, int64_t ldb, int b_mn_major,
                      int64_t m, int64_t n, int64_t k, int tile_n, float* c, int64_t ldc, const float* c_in,
                      int* status, void* stream) {
    if (a_bf16 == nullptr || b_bf16 == nullptr || c == nullptr) return fail(MECLIP_EINVAL, "debug_gemm: null pointer");
    if (!aligned16(c) || ldc % 4 != 0 || n % 8 != 0) return fail(MECLIP_EINVAL, "debug_gemm: c must be 16-byte aligned, n a multiple of 8");
    int rc = check_device();
    if (rc) return rc;
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.out = c;
    p.ld_out = ldc;
    p.out_bf16 = 0;
    p.acc_in = c_in;
    p.ld_acc = ldc;
    p.status = status;
    Operand a{a_bf16, lda, a_mn_major != 0}, b{b_bf16, ldb, b_mn_major != 0};
    t_tag = TAG_DX;
    return launch_gemm(EPI_OUT, a, b, m, n, k, tile_n > 0 ? tile_n : pick_bn(n), p, (cudaStream_t)stream);
}

}  // extern "C"
