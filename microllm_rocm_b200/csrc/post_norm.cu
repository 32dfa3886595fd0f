// The step of a block that normalises a sublayer's result BEFORE adding it (norms on both sides of every sublayer), fp32:
//
//   mlb_normed_add_rmsnorm   d = s1 * sum_k d1[k][r] + s2 * sum_k d2[k][r]        (d2 optional: two mixers side by side)
//                            x[r] += d / sqrt(mean(d^2) + eps) * w_post            in place, the residual stream
//                            out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w_next     optional: the norm in front of the next
//                                                                                  sublayer, stored in the compute dtype
//
// d1/d2 may be K-split partial results, added in split order.  One block of a fixed size per row, reductions in a fixed tree: a
// row's result depends on the row alone.  Rows of up to 4,096 columns stay in registers (up to sixteen columns a thread,
// the partial results of all of them fetched side by side, both weights fetched before the wait for the predecessor: a
// decode step's few rows are all latency); wider rows are kept in shared memory between the passes.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int PN_THREADS = 256;

struct PostNormParams {
    float* x;                 // [rows, width] fp32
    const float* d1; int n1; long long stride1; float s1;
    const float* d2; int n2; long long stride2; float s2;
    const float* w_post; const float* w_next;
    void* out;                // compute dtype, may be null (then w_next is unused)
    int width; float eps;
};

__device__ __forceinline__ float partial_sum(const float* at, int n, long long stride) {
    float v = at[0];
    for (int k = 1; k < n; ++k) v += at[(size_t)k * stride];
    return v;
}

template <typename OutT>
__global__ void __launch_bounds__(PN_THREADS) normed_add_rmsnorm_kernel(PostNormParams p) {
    pdl_prologue();
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[32];
    const int W = p.width;
    const size_t r = blockIdx.x;
    float* xr = p.x + r * W;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) {
        float d = p.s1 * partial_sum(p.d1 + r * W + c, p.n1, p.stride1);
        if (p.d2) d = fmaf(p.s2, partial_sum(p.d2 + r * W + c, p.n2, p.stride2), d);
        row_s[c] = d;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + p.eps);
    float ss2 = 0.0f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) {
        const float x = fmaf(row_s[c] * inv, p.w_post[c], xr[c]);
        xr[c] = x;
        row_s[c] = x;
        ss2 = fmaf(x, x, ss2);
    }
    if (!p.out) return;
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)W + p.eps);
    OutT* yr = (OutT*)p.out + r * W;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) yr[c] = from_f32<OutT>(row_s[c] * inv2 * p.w_next[c]);
}

// The row in registers: column threadIdx.x + 256 i is element i of a thread.  The order of every sum is that of the kernel above.
template <typename OutT, int PER>
__global__ void __launch_bounds__(PN_THREADS) normed_add_rmsnorm_reg_kernel(PostNormParams p) {
    __shared__ float scratch[32];
    const int W = p.width;
    const size_t r = blockIdx.x;
    float wp[PER], wn[PER];
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < PER; ++i) {            // weights: no kernel of a step writes them
        const int c = threadIdx.x + i * PN_THREADS;
        wp[i] = c < W ? p.w_post[c] : 0.0f;
        wn[i] = (p.out && c < W) ? p.w_next[c] : 0.0f;
    }
    pdl_wait();
    float* xr = p.x + r * W;
    float x[PER], d[PER], e[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * PN_THREADS;
        x[i] = c < W ? xr[c] : 0.0f;
        d[i] = c < W ? p.d1[r * W + c] : 0.0f;
        e[i] = (p.d2 && c < W) ? p.d2[r * W + c] : 0.0f;
    }
    for (int k = 1; k < p.n1; ++k) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = threadIdx.x + i * PN_THREADS;
            if (c < W) d[i] += p.d1[(size_t)k * p.stride1 + r * W + c];
        }
    }
    if (p.d2) {
        for (int k = 1; k < p.n2; ++k) {
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int c = threadIdx.x + i * PN_THREADS;
                if (c < W) e[i] += p.d2[(size_t)k * p.stride2 + r * W + c];
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        d[i] = p.s1 * d[i];
        if (p.d2) d[i] = fmaf(p.s2, e[i], d[i]);
        ss = fmaf(d[i], d[i], ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + p.eps);
    float ss2 = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * PN_THREADS;
        x[i] = fmaf(d[i] * inv, wp[i], x[i]);
        if (c < W) xr[c] = x[i];
        ss2 = fmaf(x[i], x[i], ss2);
    }
    if (!p.out) return;
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)W + p.eps);
    OutT* yr = (OutT*)p.out + r * W;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * PN_THREADS;
        if (c < W) yr[c] = from_f32<OutT>(x[i] * inv2 * wn[i]);
    }
}

template <typename OutT>
int launch_in_registers(const PostNormParams& p, int rows, cudaStream_t stream) {
    const int per = (p.width + PN_THREADS - 1) / PN_THREADS;
    if (per <= 1) launch_kernel(normed_add_rmsnorm_reg_kernel<OutT, 1>, (unsigned)rows, PN_THREADS, 0, stream, p);
    else if (per <= 2) launch_kernel(normed_add_rmsnorm_reg_kernel<OutT, 2>, (unsigned)rows, PN_THREADS, 0, stream, p);
    else if (per <= 4) launch_kernel(normed_add_rmsnorm_reg_kernel<OutT, 4>, (unsigned)rows, PN_THREADS, 0, stream, p);
    else if (per <= 8) launch_kernel(normed_add_rmsnorm_reg_kernel<OutT, 8>, (unsigned)rows, PN_THREADS, 0, stream, p);
    else launch_kernel(normed_add_rmsnorm_reg_kernel<OutT, 16>, (unsigned)rows, PN_THREADS, 0, stream, p);
    return check_launch("normed_add_rmsnorm");
}

}  // namespace

MLB_EXPORT int mlb_normed_add_rmsnorm(float* x, const float* d1, int n1, long long stride1, float s1, const float* d2, int n2,
                                      long long stride2, float s2, const float* w_post, const float* w_next, void* out,
                                      int out_dtype, int rows, int width, float eps, cudaStream_t stream) {
    if (rows < 0 || width <= 0 || !x || !d1 || n1 < 1 || (d2 && n2 < 1) || !w_post || (out && !w_next))
        return fail(MLB_INVALID_ARGUMENT, "normed_add_rmsnorm: bad operands");
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return fail(MLB_UNSUPPORTED_SIZE, "normed_add_rmsnorm: width %d", width);
    if (rows == 0) return MLB_OK;
    PostNormParams p{x, d1, n1, stride1, s1, d2, n2, stride2, s2, w_post, w_next, out, width, eps};
    auto go = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "normed_add_rmsnorm: cannot reserve %zu bytes of shared memory", smem);
        }
        launch_kernel(kernel, (unsigned)rows, PN_THREADS, smem, stream, p);
        return check_launch("normed_add_rmsnorm");
    };
    if (out && out_dtype != MLB_F32 && out_dtype != MLB_BF16) return fail(MLB_INVALID_ARGUMENT, "normed_add_rmsnorm: unknown output dtype %d", out_dtype);
    if (width <= 16 * PN_THREADS)
        return (!out || out_dtype == MLB_F32) ? launch_in_registers<float>(p, rows, stream) : launch_in_registers<__nv_bfloat16>(p, rows, stream);
    if (!out || out_dtype == MLB_F32) return go(normed_add_rmsnorm_kernel<float>);
    if (out_dtype == MLB_BF16) return go(normed_add_rmsnorm_kernel<__nv_bfloat16>);
    return fail(MLB_INVALID_ARGUMENT, "normed_add_rmsnorm: unknown output dtype %d", out_dtype);
}
