// Softmax attention whose keys and values may have different widths, with the steps that come between the
// projections and the scores:
//
//   mlb_row_norm_columns    sums the K-split partial results of a projection into plain fp32 rows and divides up to two
//                           blocks of columns (all of q, all of k) by their root mean square over the WHOLE block,
//                           times a weight of the block's length: a norm in front of the split into heads.
//   mlb_qk_prepare          a bias per projection column (optional); per head: rms norm of q and k, each with a weight shared by the heads or with none (optional;
//                           `norm_where` 1: in front of the rotation, 2: behind it), rotation of the first `rot_dims`
//                           elements in interleaved pairs (2i, 2i + 1) by position * freq[i] with cos and sin times
//                           `magnitude` (optional), q times 1 + coef * ln(floor((pos + 1) / every) + 1) (optional);
//                           q goes out in the compute dtype, k and v into the pages.  v may be the projected k itself.
//   mlb_paged_attention_kv  plain attention over those pages: one warp per (query token, query head), keys in tiles of
//                           32 at absolute multiples of 32 with a running maximum and sum (the order of every addition
//                           depends on the position alone, not on how the tokens were cut into steps), optional window,
//                           optional output gate: o * sigmoid(gate) with the gate read from a projection's fp32 output
//                           (one gate per element of a head, or one per head); optional cap on the scores,
//                           s <- cap * tanh(s / cap); optional sink: exp(sink[head]) joins the softmax's denominator
//                           (no key, no value, neither scaled nor capped).
//
// A page holds the keys of every kv head [NKV, page_size, DK] and behind them the values [NKV, page_size, DV].
// Everything here is fp32 arithmetic; the inputs are fp32 columns of a projection's output (or K-split partial
// results, summed in split order).
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;
constexpr int PER_LANE = MAX_D / 32;

struct Columns {               // a block of columns of fp32 rows, possibly K-split partial results
    const float* base; long long ld; int n_partials; long long partial_stride;
    __device__ __forceinline__ float at(long long row, int col) const {
        const float* p = base + row * ld + col;
        float v = p[0];
        for (int k = 1; k < n_partials; ++k) v += p[(size_t)k * partial_stride];
        return v;
    }
};

struct PrepareParams {
    Columns q, k, v;           // q: H * DK columns from q_col, k: G * DK, v: G * DV (v may alias k's columns)
    int q_col, k_col, v_col;
    const float* q_norm; const float* k_norm; float eps;
    int norm_where;            // 0: no norm, 1: before the rotation, 2: after it (a null weight: the plain quotient)
    const float* freq; int rot_dims; float magnitude;
    float temp_coef; int temp_every;
    const int* positions; const int* token_seq; const int* block_table;
    int max_blocks, num_pages, page_size;
    void* q_out;               // [T, H * DK]
    void* pages;
    int T, H, G, DK, DV;
    int PK, PV;                // widths of a stored query / key row and of a stored value row (>= DK, DV; the rest is zero)
    const float* bias;         // one per column of the projection that q (and k, v when they share its rows) come from; null: none
    int* error_flag;
};

// NL: elements a lane holds (the widest stored row is at most 32 * NL elements)
template <typename OutT, typename KVT, int NL>
__global__ void __launch_bounds__(WARPS * 32) qk_prepare_kernel(PrepareParams p) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = p.H + 2 * p.G;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * items) return;
    const int t = (int)(item / items), which = (int)(item % items);
    const int pos = p.positions[t];
    const bool is_q = which < p.H, is_k = !is_q && which < p.H + p.G;
    const int head = is_q ? which : (is_k ? which - p.H : which - p.H - p.G);
    const int D = (is_q || is_k) ? p.DK : p.DV;
    const int P = (is_q || is_k) ? p.PK : p.PV;       // stored width
    if (!is_q && !p.pages) return;
    // the row's elements first: their loads need nothing of the page lookup below and travel while it runs
    const Columns& src = is_q ? p.q : (is_k ? p.k : p.v);
    const int col = (is_q ? p.q_col : (is_k ? p.k_col : p.v_col)) + head * D;
    float x[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        const int c = lane + 32 * i;
        x[i] = c < D ? src.at(t, col + c) + (p.bias ? p.bias[col + c] : 0.0f) : 0.0f;
    }
    // where the item goes
    KVT* page_row = nullptr;
    if (!is_q) {
        const int seq = p.token_seq[t];
        const int block = pos / p.page_size;
        const int page = block < p.max_blocks ? p.block_table[(size_t)seq * p.max_blocks + block] : -1;
        if (page < 0 || page >= p.num_pages) {
            if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 1);
            return;
        }
        const size_t page_stride = (size_t)p.G * p.page_size * (p.PK + p.PV);
        const size_t within = is_k ? ((size_t)head * p.page_size + pos % p.page_size) * p.PK
                                   : (size_t)p.G * p.page_size * p.PK + ((size_t)head * p.page_size + pos % p.page_size) * p.PV;
        page_row = (KVT*)p.pages + (size_t)page * page_stride + within;
    }
    if (is_q || is_k) {
        const float* w = is_q ? p.q_norm : p.k_norm;
        auto norm = [&]() {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < NL; ++i) ss = fmaf(x[i], x[i], ss);
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.eps);
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                if (c < D) x[i] = w ? x[i] * inv * w[c] : x[i] * inv;
            }
        };
        if (p.norm_where == 1) norm();
        if (p.freq && p.rot_dims > 0) {
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                const float other = __shfl_xor_sync(0xffffffffu, x[i], 1);     // the pair's other element sits in the next lane
                if (c < p.rot_dims) {
                    const float angle = (float)pos * p.freq[c >> 1];
                    const float cs = cosf(angle) * p.magnitude, sn = sinf(angle) * p.magnitude;
                    x[i] = (c & 1) ? x[i] * cs + other * sn : x[i] * cs - other * sn;
                }
            }
        }
        if (p.norm_where == 2) norm();
        if (is_q && p.temp_every > 0) {
            const float temp = 1.0f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.0f);
#pragma unroll
            for (int i = 0; i < NL; ++i) x[i] *= temp;
        }
    }
    if (is_q) {
        OutT* out = (OutT*)p.q_out + ((size_t)t * p.H + head) * P;
#pragma unroll
        for (int i = 0; i < NL; ++i) { const int c = lane + 32 * i; if (c < P) out[c] = from_f32<OutT>(c < D ? x[i] : 0.0f); }
    } else {
#pragma unroll
        for (int i = 0; i < NL; ++i) { const int c = lane + 32 * i; if (c < P) page_row[c] = from_f32<KVT>(c < D ? x[i] : 0.0f); }
    }
}

struct AttnParams {
    const void* q;           // [T, NH * DK]
    const void* pages;
    void* out;               // [T, NH * DV]
    const int* positions; const int* token_seq; const int* block_table;
    int max_blocks, num_pages, page_size;
    int tokens, num_heads, num_kv_heads, dk, dv;
    int chunk;               // > 0: only keys of the query's own block of `chunk` positions (counted from 0)
    int window;              // 0: all earlier keys
    float scale;
    Columns gate; int gate_col;      // gate.base null: no gate
    int gate_per_head;               // 1: one gate per (token, head) at gate_col + head; 0: one per element at gate_col + head * dv + c
    const float* sink;               // [heads] or null: exp(sink[head]) joins the denominator
    float softcap;                   // > 0: s <- softcap * tanh(s / softcap)
    int* error_flag;
};

__device__ __forceinline__ float sigmoid_f32(float g) { return g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g)); }

template <typename QT, typename KVT, typename OutT>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kv_kernel(AttnParams p) {
    pdl_prologue();
    __shared__ float q_s[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.tokens * p.num_heads) return;
    const int t = (int)(item / p.num_heads), h = (int)(item % p.num_heads);
    const int DK = p.dk, DV = p.dv;
    const int kvh = h / (p.num_heads / p.num_kv_heads);
    const int pos = p.positions[t];
    const int seq = p.token_seq[t];
    const int lo = first_visible_key(pos, p.window, p.chunk);

    const QT* qrow = (const QT*)p.q + ((size_t)t * p.num_heads + h) * DK;
    for (int c = lane; c < DK; c += 32) q_s[warp][c] = to_f32(qrow[c]);
    __syncwarp();

    float acc[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const size_t page_stride = (size_t)p.num_kv_heads * p.page_size * (DK + DV);
    const size_t v_base = (size_t)p.num_kv_heads * p.page_size * DK;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int kp = base + lane;
        bool valid = kp >= lo && kp <= pos;
        long long k_off = -1, v_off = -1;
        if (valid) {
            const int block = kp / p.page_size;
            const int page = block < p.max_blocks ? table[block] : -1;
            if (page < 0 || page >= p.num_pages) {
                if (p.error_flag) atomicExch(p.error_flag, 2);
                valid = false;
            } else {
                const size_t row = (size_t)kvh * p.page_size + kp % p.page_size;
                k_off = (long long)((size_t)page * page_stride + row * DK);
                v_off = (long long)((size_t)page * page_stride + v_base + row * DV);
            }
        }
        float s = -INFINITY;
        if (valid) {
            const KVT* krow = (const KVT*)p.pages + k_off;
            float dot = 0.0f;
            for (int c = 0; c < DK; ++c) dot = fmaf(q_s[warp][c], to_f32(krow[c]), dot);
            s = dot * p.scale;
            if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float prob = valid ? expf(s - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(prob);
        m = m_new;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) acc[i] *= corr;
        const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, prob, j);
            const long long off_j = __shfl_sync(0xffffffffu, v_off, j);
            if (!((valid_mask >> j) & 1u)) continue;
            const KVT* vrow = (const KVT*)p.pages + off_j;
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const int c = lane + 32 * i;
                if (c < DV) acc[i] = fmaf(pj, to_f32(vrow[c]), acc[i]);
            }
        }
    }
    OutT* orow = (OutT*)p.out + ((size_t)t * p.num_heads + h) * DV;
    float shrink = 1.0f;
    if (p.sink) {
        // the sink joins last: with m' = max(m, sink), l' = l * exp(m - m') + exp(sink - m') and the sums shrink alike
        const float sk = p.sink[h];
        const float m_new = fmaxf(m, sk);
        shrink = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * shrink + expf(sk - m_new);
    }
    const float inv = l > 0.0f ? shrink / l : 0.0f;
    const float head_gate = (p.gate.base && p.gate_per_head) ? sigmoid_f32(p.gate.at(t, p.gate_col + h)) : 1.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < DV) {
            float o = acc[i] * inv;
            if (p.gate.base) o *= p.gate_per_head ? head_gate : sigmoid_f32(p.gate.at(t, p.gate_col + h * DV + c));
            orow[c] = from_f32<OutT>(o);
        }
    }
}

// out[t, h * DV + c] = o[t, h * PV + c] * sigmoid(gate[t, gate_col + h * DV + c]): the heads' outputs taken out of rows
// that are wider than a value (an attention kernel that ran on padded heads) and gated.  gate.base null: no gate.
struct GateParams {
    const void* o; void* out; Columns gate; int gate_col; int T, H, DV, PV; int gate_per_head;
};

template <typename T>
__global__ void gate_heads_kernel(GateParams p) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = (long long)p.T * p.H * p.DV;
    if (i >= n) return;
    const int c = (int)(i % p.DV), h = (int)((i / p.DV) % p.H);
    const long long t = i / ((long long)p.DV * p.H);
    float o = to_f32(((const T*)p.o)[(t * p.H + h) * p.PV + c]);
    if (p.gate.base) o *= sigmoid_f32(p.gate.at(t, p.gate_per_head ? p.gate_col + h : p.gate_col + h * p.DV + c));
    ((T*)p.out)[i] = from_f32<T>(o);
}

// out[t, c] = sum of the partial results at (t, c); columns [col_a, col_a + n_a) and [col_b, col_b + n_b) are then divided by the
// root mean square over their own block and multiplied by w_a / w_b (null: no weight).  n_b may be 0.  One CTA per row, a
// fixed number of threads: a row's sums never depend on the batch.
constexpr int ROW_NORM_THREADS = 256;
__global__ void __launch_bounds__(ROW_NORM_THREADS)
row_norm_columns_kernel(Columns src, int cols, int col_a, int n_a, const float* __restrict__ w_a, int col_b, int n_b,
                        const float* __restrict__ w_b, float eps, float* __restrict__ out) {
    pdl_prologue();
    __shared__ float scratch[32];
    const long long t = blockIdx.x;
    float* row = out + (size_t)t * cols;
    float ss_a = 0.0f, ss_b = 0.0f;
    for (int c = threadIdx.x; c < cols; c += ROW_NORM_THREADS) {
        const float v = src.at(t, c);
        row[c] = v;
        if (c >= col_a && c < col_a + n_a) ss_a = fmaf(v, v, ss_a);
        if (c >= col_b && c < col_b + n_b) ss_b = fmaf(v, v, ss_b);
    }
    const float inv_a = 1.0f / sqrtf(block_sum(ss_a, scratch) / (float)n_a + eps);
    const float inv_b = n_b > 0 ? 1.0f / sqrtf(block_sum(ss_b, scratch) / (float)n_b + eps) : 0.0f;
    for (int c = threadIdx.x; c < cols; c += ROW_NORM_THREADS) {        // every thread rewrites only what it wrote itself
        if (c >= col_a && c < col_a + n_a) row[c] = w_a ? row[c] * inv_a * w_a[c - col_a] : row[c] * inv_a;
        else if (c >= col_b && c < col_b + n_b) row[c] = w_b ? row[c] * inv_b * w_b[c - col_b] : row[c] * inv_b;
    }
}


// The same for bf16 rows whose widths are multiples of 8: a thread moves 8 elements of one head (16 bytes); with one gate per
// head it reads that gate once.
__global__ void gate_heads_x8_kernel(GateParams p) {
    pdl_prologue();
    const int per_head = p.DV / 8, per_token = p.H * per_head;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.T * per_token) return;
    const long long t = i / per_token;
    const int rest = (int)(i % per_token), h = rest / per_head, c = (rest % per_head) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.o + (t * p.H + h) * p.PV + c);
    if (p.gate.base) {
        __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&raw);
        const float head_gate = p.gate_per_head ? sigmoid_f32(p.gate.at(t, p.gate_col + h)) : 1.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 v = __bfloat1622float2(pair[k]);
            if (p.gate_per_head) { v.x *= head_gate; v.y *= head_gate; }
            else {
                v.x *= sigmoid_f32(p.gate.at(t, p.gate_col + h * p.DV + c + 2 * k));
                v.y *= sigmoid_f32(p.gate.at(t, p.gate_col + h * p.DV + c + 2 * k + 1));
            }
            pair[k] = __floats2bfloat162_rn(v.x, v.y);
        }
    }
    *reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + (t * p.H + h) * p.DV + c) = raw;
}

}  // namespace

MLB_EXPORT int mlb_row_norm_columns(const float* src, long long ld, int n_partials, long long partial_stride, int T, int cols,
                                    int col_a, int n_a, const float* w_a, int col_b, int n_b, const float* w_b, float eps,
                                    float* out, cudaStream_t stream) {
    if (T < 0 || cols <= 0 || ld < cols || n_partials < 1 || n_a <= 0 || col_a < 0 || col_a + n_a > cols || n_b < 0 || col_b < 0 ||
        col_b + n_b > cols || !src || !out)
        return fail(MLB_INVALID_ARGUMENT, "row_norm_columns: bad sizes");
    if (T == 0) return MLB_OK;
    launch_kernel(row_norm_columns_kernel, (unsigned)T, ROW_NORM_THREADS, 0, stream, Columns{src, ld, n_partials, partial_stride}, cols,
                  col_a, n_a, w_a, col_b, n_b, w_b, eps, out);
    return check_launch("row_norm_columns");
}

MLB_EXPORT int mlb_gate_heads(const void* o, void* out, int dtype, const float* gate, long long gate_ld, int gate_partials,
                              long long gate_partial_stride, int gate_col, int T, int H, int DV, int stored_v, int gate_per_head,
                              cudaStream_t stream) {
    if (T < 0 || H <= 0 || DV <= 0 || stored_v < DV || !o || !out) return fail(MLB_INVALID_ARGUMENT, "gate_heads: bad operands");
    if (T == 0) return MLB_OK;
    GateParams p{o, out, Columns{gate, gate_ld, gate_partials < 1 ? 1 : gate_partials, gate_partial_stride}, gate_col, T, H, DV, stored_v,
                 gate_per_head ? 1 : 0};
    const long long n = (long long)T * H * DV;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == MLB_BF16 && DV % 8 == 0 && stored_v % 8 == 0 && ((uintptr_t)o | (uintptr_t)out) % 16 == 0)
        launch_kernel(gate_heads_x8_kernel, (unsigned)((n / 8 + 255) / 256), 256, 0, stream, p);
    else if (dtype == MLB_BF16) launch_kernel(gate_heads_kernel<__nv_bfloat16>, blocks, 256, 0, stream, p);
    else if (dtype == MLB_F32) launch_kernel(gate_heads_kernel<float>, blocks, 256, 0, stream, p);
    else return fail(MLB_INVALID_ARGUMENT, "gate_heads: unsupported dtype %d", dtype);
    return check_launch("gate_heads");
}

MLB_EXPORT int mlb_qk_prepare(const float* src, long long ld, int n_partials, long long partial_stride, int q_col, int k_col,
                              int v_col, const float* kv_src, long long kv_ld, int kv_partials, long long kv_partial_stride,
                              const float* q_norm, const float* k_norm, float eps, int norm_where, const float* freq, int rot_dims,
                              float magnitude, float temp_coef, int temp_every, const int* positions, const int* token_seq,
                              const int* block_table, int max_blocks, int num_pages, int page_size, void* q_out, int q_dtype,
                              void* pages, int kv_dtype, int T, int H, int G, int DK, int DV, int stored_k, int stored_v,
                              const float* bias, int* error_flag, cudaStream_t stream) {
    // `src` holds q (and k, v when kv_src is null); `kv_src`, when given, holds k and v (a projection that went through
    // another kernel first: the raw values of "values are the projected keys" come from the same place as k)
    if (T < 0 || H <= 0 || G <= 0 || H % G || DK <= 0 || DV <= 0 || DK > MAX_D || DV > MAX_D)
        return fail(MLB_UNSUPPORTED_SIZE, "qk_prepare: heads %d/%d, widths %d/%d (at most %d)", H, G, DK, DV, MAX_D);
    if (stored_k < DK || stored_v < DV || stored_k > MAX_D || stored_v > MAX_D)
        return fail(MLB_INVALID_ARGUMENT, "qk_prepare: stored widths %d/%d for %d/%d (at most %d)", stored_k, stored_v, DK, DV, MAX_D);
    if (norm_where < 0 || norm_where > 2) return fail(MLB_INVALID_ARGUMENT, "qk_prepare: norm_where %d", norm_where);
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > DK) return fail(MLB_INVALID_ARGUMENT, "qk_prepare: rot_dims %d of %d", rot_dims, DK);
    if (pages && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !block_table))
        return fail(MLB_INVALID_ARGUMENT, "qk_prepare: bad cache geometry");
    if (bias && kv_src) return fail(MLB_INVALID_ARGUMENT, "qk_prepare: a bias belongs to one projection's columns");
    if (T == 0) return MLB_OK;
    PrepareParams p{};
    p.q = Columns{src, ld, n_partials, partial_stride};
    p.k = p.v = kv_src ? Columns{kv_src, kv_ld, kv_partials, kv_partial_stride} : p.q;
    p.q_col = q_col; p.k_col = k_col; p.v_col = v_col;
    p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps; p.norm_where = norm_where; p.freq = freq; p.rot_dims = rot_dims; p.magnitude = magnitude;
    p.temp_coef = temp_coef; p.temp_every = temp_every; p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
    p.max_blocks = max_blocks; p.num_pages = num_pages; p.page_size = page_size; p.q_out = q_out; p.pages = pages;
    p.T = T; p.H = H; p.G = G; p.DK = DK; p.DV = DV; p.PK = stored_k; p.PV = stored_v; p.bias = bias; p.error_flag = error_flag;
    const long long items = (long long)T * (H + 2 * G);
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const int kvd = pages ? kv_dtype : q_dtype;
    const int widest = stored_k > stored_v ? stored_k : stored_v;
    auto go = [&](auto k1, auto k2, auto k4, auto k8) {
        if (widest <= 32) launch_kernel(k1, blocks, WARPS * 32, 0, stream, p);
        else if (widest <= 64) launch_kernel(k2, blocks, WARPS * 32, 0, stream, p);
        else if (widest <= 128) launch_kernel(k4, blocks, WARPS * 32, 0, stream, p);
        else launch_kernel(k8, blocks, WARPS * 32, 0, stream, p);
    };
    typedef __nv_bfloat16 bf;
    if (q_dtype == MLB_F32 && kvd == MLB_F32)
        go(qk_prepare_kernel<float, float, 1>, qk_prepare_kernel<float, float, 2>, qk_prepare_kernel<float, float, 4>, qk_prepare_kernel<float, float, 8>);
    else if (q_dtype == MLB_BF16 && kvd == MLB_BF16)
        go(qk_prepare_kernel<bf, bf, 1>, qk_prepare_kernel<bf, bf, 2>, qk_prepare_kernel<bf, bf, 4>, qk_prepare_kernel<bf, bf, 8>);
    else if (q_dtype == MLB_F32 && kvd == MLB_BF16)
        go(qk_prepare_kernel<float, bf, 1>, qk_prepare_kernel<float, bf, 2>, qk_prepare_kernel<float, bf, 4>, qk_prepare_kernel<float, bf, 8>);
    else return fail(MLB_INVALID_ARGUMENT, "qk_prepare: unsupported dtypes %d/%d", q_dtype, kv_dtype);
    return check_launch("qk_prepare");
}

MLB_EXPORT int mlb_paged_attention_kv(const void* q, int q_dtype, const void* pages, int kv_dtype, void* out, int out_dtype,
                                      const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                                      int num_pages, int page_size, int tokens, int num_heads, int num_kv_heads, int dk, int dv,
                                      int window, int chunk, float scale, const float* gate, long long gate_ld, int gate_partials,
                                      long long gate_partial_stride, int gate_col, int gate_per_head, const float* sink, float softcap,
                                      int* error_flag, cudaStream_t stream) {
    if (tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_kv: bad head counts %d/%d", num_heads, num_kv_heads);
    if (dk <= 0 || dk > MAX_D || dv <= 0 || dv > MAX_D)
        return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_kv: widths %d/%d not in 1..%d", dk, dv, MAX_D);
    if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || chunk < 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_kv: bad cache geometry");
    if (tokens == 0) return MLB_OK;
    AttnParams p{q, pages, out, positions, token_seq, block_table, max_blocks, num_pages, page_size, tokens, num_heads,
                 num_kv_heads, dk, dv, chunk, window, scale, Columns{gate, gate_ld, gate_partials < 1 ? 1 : gate_partials, gate_partial_stride},
                 gate_col, gate_per_head ? 1 : 0, sink, softcap, error_flag};
    if (softcap < 0.0f) return fail(MLB_INVALID_ARGUMENT, "paged_attention_kv: a cap on the scores is positive (0: none)");
    const long long items = (long long)tokens * num_heads;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (q_dtype == MLB_F32 && kv_dtype == MLB_F32 && out_dtype == MLB_F32)
        launch_kernel(paged_attention_kv_kernel<float, float, float>, blocks, WARPS * 32, 0, stream, p);
    else if (q_dtype == MLB_BF16 && kv_dtype == MLB_BF16 && out_dtype == MLB_BF16)
        launch_kernel(paged_attention_kv_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_kv: unsupported dtypes %d/%d/%d", q_dtype, kv_dtype, out_dtype);
    return check_launch("paged_attention_kv");
}
