// Residual-stream kernels of decoders whose blocks scale what they add:
//
//   embed_gather_scaled   out[t,:] = table[id[t],:] * scale               (bad id -> NaN)
//   add_table_rows        x[t,:] += table[index[t],:]                     learned additive positions
//   add_scaled_rmsnorm    x[t,:] += s[:] * sum_k delta_k[t,:];  out[t,:] = x[t,:] / sqrt(mean(x^2) + eps) * w[:]
//   add_scaled_inplace    x[t,:] += s[:] * sum_k delta_k[t,:]
//   stream_entry          x[t,:] += (x0 ? x0[t,:] : 0) + v[:]             what a pass of looped layers adds first
//
//   bigram_add            x[t,:] += table[row(t),:], row = (previous token * a + token * b) mod n, or row n for a sequence's
//                         first token; the previous token of a step's first token is the sequence's state (one int per slot).
//                         Given the token table as well, x[t,:] = tokens[id[t],:] + table[row(t),:] in one pass (bad id -> NaN).
//   bigram_state          state[slot of a] = the last token sequence a brought in this step
//   softcap_rows          x <- cap * tanh(x / cap) in place
//
// `s` is a per-column factor (a layer scale times the block's residual multiplier), null for none.  All sums are
// fp32; one block per row with a fixed number of threads, so that a row's result never depends on the batch.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int ROW_THREADS = 256;

template <typename TableT>
__global__ void embed_scaled_kernel(const TableT* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                    int tokens, int width, int vocab, float scale) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int id = ids[t];
    float* dst = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
        return;
    }
    const TableT* src = table + (size_t)id * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = to_f32(src[c]) * scale;
}

template <typename TableT>
__global__ void add_table_rows_kernel(float* __restrict__ x, const TableT* __restrict__ table, const int* __restrict__ index,
                                      int tokens, int width, int rows) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int r = index[t];
    float* dst = x + (size_t)t * width;
    if (r < 0 || r >= rows) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
        return;
    }
    const TableT* src = table + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] += to_f32(src[c]);
}

__device__ __forceinline__ float delta_sum(const float* delta, int n_delta, long long stride, size_t at) {
    float d = delta[at];
    for (int k = 1; k < n_delta; ++k) d += delta[(size_t)k * stride + at];
    return d;
}

template <typename OutT>
__global__ void __launch_bounds__(ROW_THREADS)
add_scaled_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                          const float* __restrict__ col_scale, const float* __restrict__ weight, OutT* __restrict__ out,
                          int width, float eps) {
    pdl_prologue();
    __shared__ float scratch[32];
    const size_t row = (size_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
        float d = delta_sum(delta, n_delta, delta_stride, row + c);
        if (col_scale) d *= col_scale[c];
        const float v = x[row + c] + d;
        x[row + c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) out[row + c] = from_f32<OutT>(x[row + c] * inv * weight[c]);
}

__global__ void add_scaled_inplace_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta,
                                          long long delta_stride, const float* __restrict__ col_scale, int width, size_t n) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = delta_sum(delta, n_delta, delta_stride, i);
    if (col_scale) d *= col_scale[i % width];
    x[i] += d;
}

__global__ void stream_entry_kernel(float* __restrict__ x, const float* __restrict__ x0, const float* __restrict__ v,
                                    int width, size_t n) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = x[i];
    if (x0) a += x0[i];
    x[i] = a + v[i % width];
}

}  // namespace

MLB_EXPORT int mlb_embed_gather_scaled(const void* table, int table_dtype, const int* ids, float* out, int tokens, int width,
                                       int vocab, float scale, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || vocab <= 0) return fail(MLB_INVALID_ARGUMENT, "embed_gather_scaled: bad sizes");
    if (tokens == 0) return MLB_OK;
    if (table_dtype == MLB_F32)
        launch_kernel(embed_scaled_kernel<float>, tokens, ROW_THREADS, 0, stream, (const float*)table, ids, out, tokens, width, vocab, scale);
    else if (table_dtype == MLB_BF16)
        launch_kernel(embed_scaled_kernel<__nv_bfloat16>, tokens, ROW_THREADS, 0, stream, (const __nv_bfloat16*)table, ids, out, tokens, width, vocab, scale);
    else
        return fail(MLB_INVALID_ARGUMENT, "embed_gather_scaled: unknown table dtype %d", table_dtype);
    return check_launch("embed_gather_scaled");
}

MLB_EXPORT int mlb_add_table_rows(float* x, const void* table, int table_dtype, const int* index, int tokens, int width,
                                  int rows, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || rows <= 0) return fail(MLB_INVALID_ARGUMENT, "add_table_rows: bad sizes");
    if (tokens == 0) return MLB_OK;
    if (table_dtype == MLB_F32)
        launch_kernel(add_table_rows_kernel<float>, tokens, ROW_THREADS, 0, stream, x, (const float*)table, index, tokens, width, rows);
    else if (table_dtype == MLB_BF16)
        launch_kernel(add_table_rows_kernel<__nv_bfloat16>, tokens, ROW_THREADS, 0, stream, x, (const __nv_bfloat16*)table, index, tokens, width, rows);
    else
        return fail(MLB_INVALID_ARGUMENT, "add_table_rows: unknown table dtype %d", table_dtype);
    return check_launch("add_table_rows");
}

MLB_EXPORT int mlb_add_scaled_rmsnorm(float* residual, const float* delta, int n_delta, long long delta_stride,
                                      const float* col_scale, const float* weight, void* out, int out_dtype, int n_rows,
                                      int width, float eps, cudaStream_t stream) {
    if (n_rows < 0 || width <= 0 || !(eps > 0.0f) || !delta || n_delta < 1)
        return fail(MLB_INVALID_ARGUMENT, "add_scaled_rmsnorm: bad sizes, eps or delta");
    if (n_rows == 0) return MLB_OK;
    if (out_dtype == MLB_F32)
        launch_kernel(add_scaled_rmsnorm_kernel<float>, n_rows, ROW_THREADS, 0, stream, residual, delta, n_delta, delta_stride, col_scale, weight, (float*)out, width, eps);
    else if (out_dtype == MLB_BF16)
        launch_kernel(add_scaled_rmsnorm_kernel<__nv_bfloat16>, n_rows, ROW_THREADS, 0, stream, residual, delta, n_delta, delta_stride, col_scale, weight, (__nv_bfloat16*)out, width, eps);
    else
        return fail(MLB_INVALID_ARGUMENT, "add_scaled_rmsnorm: unknown output dtype %d", out_dtype);
    return check_launch("add_scaled_rmsnorm");
}

MLB_EXPORT int mlb_add_scaled_inplace(float* x, const float* delta, int n_delta, long long delta_stride, const float* col_scale,
                                      int width, long long n, cudaStream_t stream) {
    if (n < 0 || n_delta < 1 || width <= 0) return fail(MLB_INVALID_ARGUMENT, "add_scaled_inplace: bad sizes");
    if (n == 0) return MLB_OK;
    launch_kernel(add_scaled_inplace_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, delta, n_delta, delta_stride, col_scale, width, (size_t)n);
    return check_launch("add_scaled_inplace");
}

MLB_EXPORT int mlb_stream_entry(float* x, const float* x0, const float* v, int width, long long n, cudaStream_t stream) {
    if (n < 0 || width <= 0 || !v) return fail(MLB_INVALID_ARGUMENT, "stream_entry: bad sizes");
    if (n == 0) return MLB_OK;
    launch_kernel(stream_entry_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, x0, v, width, (size_t)n);
    return check_launch("stream_entry");
}

namespace {

template <typename TableT>
__global__ void bigram_add_kernel(float* __restrict__ x, const TableT* __restrict__ table, const TableT* __restrict__ token_table, int vocab,
                                  const int* __restrict__ ids,
                                  const int* __restrict__ token_seq, const int* __restrict__ seq_starts, const int* __restrict__ seq_pos0,
                                  const int* __restrict__ state, const int* __restrict__ slots, int num_slots, int tokens, int width,
                                  int buckets, long long mul_prev, long long mul_cur, int* __restrict__ error_flag) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int seq = token_seq[t];
    long long prev = -1;
    if (t > seq_starts[seq]) prev = ids[t - 1];
    else if (seq_pos0[seq] > 0) {
        const int slot = slots[seq];
        if (slot < 0 || slot >= num_slots) {
            if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 4);
            return;
        }
        prev = state[slot];
    }
    const int row = prev < 0 ? buckets : (int)((prev * mul_prev + (long long)ids[t] * mul_cur) % buckets);
    const TableT* src = table + (size_t)row * width;
    float* dst = x + (size_t)t * width;
    if (token_table) {
        const int id = ids[t];
        if (id < 0 || id >= vocab) {
            for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
            return;
        }
        const TableT* own = token_table + (size_t)id * width;
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = to_f32(own[c]) + to_f32(src[c]);
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] += to_f32(src[c]);
}

__global__ void bigram_state_kernel(const int* __restrict__ ids, const int* __restrict__ seq_starts, int* __restrict__ state,
                                    const int* __restrict__ slots, int num_slots, int num_seqs) {
    pdl_prologue();
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= num_seqs) return;
    const int slot = slots[a];
    if (slot >= 0 && slot < num_slots && seq_starts[a + 1] > seq_starts[a]) state[slot] = ids[seq_starts[a + 1] - 1];
}

__global__ void softcap_rows_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace

MLB_EXPORT int mlb_bigram_add(float* x, const void* table, int table_dtype, const void* token_table, int vocab, const int* ids, const int* token_seq, const int* seq_starts,
                              const int* seq_pos0, int* state, const int* slots, int num_slots, int tokens, int num_seqs, int width,
                              int buckets, int mul_prev, int mul_cur, int update_state, int* error_flag, cudaStream_t stream) {
    if (tokens < 0 || num_seqs < 0 || width <= 0 || buckets <= 0 || num_slots <= 0 || !x || !table || !ids || !state || !slots)
        return fail(MLB_INVALID_ARGUMENT, "bigram_add: bad operands");
    if (tokens == 0) return MLB_OK;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == MLB_BF16)
        launch_kernel(bigram_add_kernel<__nv_bfloat16>, (unsigned)tokens, threads, 0, stream, x, (const __nv_bfloat16*)table,
                      (const __nv_bfloat16*)token_table, vocab, ids, token_seq,
                      seq_starts, seq_pos0, (const int*)state, slots, num_slots, tokens, width, buckets, (long long)mul_prev, (long long)mul_cur, error_flag);
    else if (table_dtype == MLB_F32)
        launch_kernel(bigram_add_kernel<float>, (unsigned)tokens, threads, 0, stream, x, (const float*)table, (const float*)token_table, vocab,
                      ids, token_seq, seq_starts,
                      seq_pos0, (const int*)state, slots, num_slots, tokens, width, buckets, (long long)mul_prev, (long long)mul_cur, error_flag);
    else return fail(MLB_INVALID_ARGUMENT, "bigram_add: unsupported table dtype %d", table_dtype);
    if (update_state)
        launch_kernel(bigram_state_kernel, (unsigned)((num_seqs + 127) / 128), 128, 0, stream, ids, seq_starts, state, slots, num_slots, num_seqs);
    return check_launch("bigram_add");
}

MLB_EXPORT int mlb_softcap_rows(float* x, long long n, float cap, cudaStream_t stream) {
    if (n < 0 || !(cap > 0.0f)) return fail(MLB_INVALID_ARGUMENT, "softcap_rows: a positive cap");
    if (n == 0) return MLB_OK;
    launch_kernel(softcap_rows_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, n, cap);
    return check_launch("softcap_rows");
}
