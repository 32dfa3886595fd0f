// Routing of tokens to experts, on the device from start to end (nothing here needs the host to know a count):
//
//   moe_select    per token, from router logits that a product left in fp32: z[e] = logits[e] + b[e]; the `top` largest
//                 (ties: the smaller index) in order of size; weights = softmax over those chosen logits only.
//                 Optionally one more column (the gate of a shared expert) whose sigmoid is stored per token.
//                 `scoring` 1: s = softmax(z) over ALL outputs (no bias inside); the `top` largest s[e] + b[e] are chosen
//                 (b a correction that only steers the choice) and the weights are the chosen s themselves, not renormalised.
//   moe_align     (below) skips, without raising the flag, ids in [experts, experts + passthrough): outputs of the router that
//                 have no expert behind them (moe_combine adds the token's own input times the weight for those).
//   moe_align     from ids[T*top] to a list of the pairs (token, choice) sorted by expert: offsets[E+1] and
//                 sorted[T*top] (pair indices); the order inside an expert is arbitrary, every pair's result is
//                 computed on its own.
//   moe_combine   out[t,:] = (sum_j w[t,j] * y[t*top + j,:] + g[t] * sum_k shared_k[t,:]) * s[:]
//                 j in order of choice; shared (may be split partial sums), g and s are optional.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int ROUTE_WARPS = 4;
constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_TOP = 32;       // one chosen logit per lane

// logits [T, ld] fp32 (or `n_partials` partial sums of a split product, `partial_stride` elements apart): columns
// 0..experts-1 are the router's, column `gate_col` (if >= 0) the pre-activation of a shared expert's gate.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_select_kernel(const float* __restrict__ logits, long long ld, int n_partials, long long partial_stride,
                  const float* __restrict__ bias, int gate_col, int tokens, int experts, int top,
                  int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ gate_out, int scoring) {
    pdl_prologue();
    extern __shared__ float logits_s[];                 // [ROUTE_WARPS][experts] (scoring 1: twice that, choice scores then s)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float* z = logits_s + (size_t)warp * experts * (scoring == 1 ? 2 : 1);
    float* score = z + experts;                         // scoring 1 only
    const float* row = logits + (size_t)t * ld;
    for (int e = lane; e < experts; e += 32) {
        float v = row[e];
        for (int k = 1; k < n_partials; ++k) v += row[(size_t)k * partial_stride + e];
        z[e] = scoring == 1 ? v : v + (bias ? bias[e] : 0.0f);
    }
    if (scoring == 1) {
        __syncwarp();
        float mx = -INFINITY;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float total = 0.0f;
        for (int e = lane; e < experts; e += 32) total += expf(z[e] - mx);
        total = warp_sum(total);
        for (int e = lane; e < experts; e += 32) {
            const float sc = expf(z[e] - mx) / total;
            score[e] = sc;
            z[e] = sc + (bias ? bias[e] : 0.0f);
        }
    }
    if (gate_col >= 0 && gate_out && lane == 0) {
        float v = row[gate_col];
        for (int k = 1; k < n_partials; ++k) v += row[(size_t)k * partial_stride + gate_col];
        gate_out[t] = 1.0f / (1.0f + expf(-v));
    }
    __syncwarp();
    // `top` rounds of a warp-wide argmax (ties: the smaller index); a chosen logit is marked by its index in `taken`
    float chosen = 0.0f, first = 0.0f, sum = 0.0f;      // lane j keeps the j-th chosen logit
    for (int j = 0; j < top; ++j) {
        float best_v = -INFINITY;
        int best = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = z[e];
            if (v != v) continue;                       // a logit that is not a number is never chosen before the others
            if (best == 0x7fffffff || v > best_v) { best = e; best_v = v; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best, o);
            if (oe != 0x7fffffff && (best == 0x7fffffff || ov > best_v || (ov == best_v && oe < best))) { best = oe; best_v = ov; }
        }
        if (best == 0x7fffffff) { best = 0; best_v = 0.0f; }      // nothing left that is a number
        if (j == 0) first = best_v;
        if (lane == (j & 31)) chosen = scoring == 1 ? score[best] : best_v;
        if (lane == 0) { ids[(size_t)t * top + j] = best; z[best] = nanf(""); }
        __syncwarp();
    }
    if (scoring == 1) {
        if (lane < top) weights[(size_t)t * top + lane] = chosen;
        return;
    }
    const float w = lane < top ? expf(chosen - first) : 0.0f;
    sum = warp_sum(w);
    if (lane < top) weights[(size_t)t * top + lane] = w / sum;
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ sorted,
                 int* __restrict__ error_flag, int passthrough) {
    pdl_prologue();
    __shared__ int count[MAX_EXPERTS];
    __shared__ int cursor[MAX_EXPERTS];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
        else if (!(e >= experts && e < experts + passthrough) && error_flag) atomicExch(error_flag, 3);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) { offsets[e] = at; cursor[e] = at; at += count[e]; }
        offsets[experts] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) sorted[atomicAdd(&cursor[e], 1)] = i;
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, const float* __restrict__ shared,
                                   int n_shared, long long shared_stride, const float* __restrict__ gate,
                                   const float* __restrict__ col_scale, float* __restrict__ out, int tokens, int width, int top,
                                   const int* __restrict__ ids, int experts, const void* __restrict__ x, int x_dtype) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float acc = 0.0f;
    if (ids) {
        // a choice at or beyond `experts` has no expert behind it: the token's own input passes, times the weight
        const float own = x_dtype == MLB_BF16 ? to_f32(((const __nv_bfloat16*)x)[i]) : ((const float*)x)[i];
        for (int j = 0; j < top; ++j) {
            const float v = ids[(size_t)t * top + j] >= experts ? own : y[((size_t)t * top + j) * width + c];
            acc = fmaf(weights[(size_t)t * top + j], v, acc);
        }
    } else
    for (int j = 0; j < top; ++j) acc = fmaf(weights[(size_t)t * top + j], y[((size_t)t * top + j) * width + c], acc);
    if (shared) {
        float s = shared[i];
        for (int k = 1; k < n_shared; ++k) s += shared[(size_t)k * shared_stride + i];
        acc += gate ? gate[t] * s : s;
    }
    out[i] = col_scale ? acc * col_scale[c] : acc;
}

}  // namespace

MLB_EXPORT int mlb_moe_select(const float* logits, long long ld, int n_partials, long long partial_stride, const float* bias,
                              int gate_col, int tokens, int experts, int top, int* ids, float* weights, float* gate_out,
                              int scoring, cudaStream_t stream) {
    if (scoring != 0 && scoring != 1) return fail(MLB_INVALID_ARGUMENT, "moe_select: unknown scoring %d", scoring);
    if (tokens < 0 || experts <= 0 || experts > MAX_EXPERTS || top <= 0 || top > experts || top > MAX_TOP || n_partials < 1 ||
        ld < experts || gate_col >= ld)
        return fail(MLB_INVALID_ARGUMENT, "moe_select: bad sizes (experts %d, top %d; at most %d and %d)", experts, top, MAX_EXPERTS, MAX_TOP);
    if (tokens == 0) return MLB_OK;
    const unsigned blocks = (tokens + ROUTE_WARPS - 1) / ROUTE_WARPS;
    launch_kernel(moe_select_kernel, blocks, ROUTE_WARPS * 32, (size_t)ROUTE_WARPS * experts * sizeof(float) * (scoring == 1 ? 2 : 1),
                  stream, logits, ld, n_partials, partial_stride, bias, gate_col, tokens, experts, top, ids, weights, gate_out, scoring);
    return check_launch("moe_select");
}

MLB_EXPORT int mlb_moe_align(const int* ids, int pairs, int experts, int* offsets, int* sorted, int* error_flag, int passthrough,
                             cudaStream_t stream) {
    if (pairs < 0 || experts <= 0 || experts > MAX_EXPERTS || passthrough < 0) return fail(MLB_INVALID_ARGUMENT, "moe_align: bad sizes");
    launch_kernel(moe_align_kernel, 1, 1024, 0, stream, ids, pairs, experts, offsets, sorted, error_flag, passthrough);
    return check_launch("moe_align");
}

MLB_EXPORT int mlb_moe_combine(const float* y, const float* weights, const float* shared, int n_shared, long long shared_stride,
                               const float* gate, const float* col_scale, float* out, int tokens, int width, int top,
                               const int* ids, int experts, const void* x, int x_dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || top <= 0 || (shared && n_shared < 1)) return fail(MLB_INVALID_ARGUMENT, "moe_combine: bad sizes");
    if (ids && (!x || (x_dtype != MLB_BF16 && x_dtype != MLB_F32))) return fail(MLB_INVALID_ARGUMENT, "moe_combine: choices without experts need the tokens' input");
    if (tokens == 0) return MLB_OK;
    const long long n = (long long)tokens * width;
    launch_kernel(moe_combine_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, y, weights, shared, n_shared, shared_stride,
                  gate, col_scale, out, tokens, width, top, ids, experts, x, x_dtype);
    return check_launch("moe_combine");
}
