// The step of a block that normalises a sublayer's result BEFORE adding it (norms on both sides of every sublayer), fp32:
//
//   mlb_normed_add_rmsnorm   d = s1 * sum_k d1[k][r] + s2 * sum_k d2[k][r]        (d2 optional: two mixers side by side)
//                            x[r] += d / sqrt(mean(d^2) + eps) * w_post            in place, the residual stream
//                            out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w_next     optional: the norm in front of the next
//                                                                                  sublayer, stored in the compute dtype
//
// d1/d2 may be K-split partial results, added in split order.  One block of a fixed size per row, the row kept in shared
// memory between the passes, reductions in a fixed tree: a row's result depends on the row alone.
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
    if (!out || out_dtype == MLB_F32) return go(normed_add_rmsnorm_kernel<float>);
    if (out_dtype == MLB_BF16) return go(normed_add_rmsnorm_kernel<__nv_bfloat16>);
    return fail(MLB_INVALID_ARGUMENT, "normed_add_rmsnorm: unknown output dtype %d", out_dtype);
}
