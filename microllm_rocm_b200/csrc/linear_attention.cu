// What surrounds a linear recurrence with a decay per key channel (the scan itself is mlb_linear_scan in delta_rule.cu).
// fp32 arithmetic throughout; only what a product reads next is stored in the compute dtype.
//
//   mlb_token_shift        y_s[t] = x[t] + (x[t-1] - x[t]) * mu_s   for s = 0..n_mix-1: every projection of a mixer reads its
//                          own blend of a token's input and the previous token's.  x[t-1] of a step's first token is the
//                          sequence's state row (zeros at position 0).
//   mlb_token_shift_state  the state row becomes the input of the step's last token (a kernel of its own behind the first:
//                          every blend of the step reads the old state).
//   mlb_decay_prepare      q * q_scale, k, v gathered out of projections' fp32 outputs (K-split partial results are summed in
//                          split order) and the decay of every (token, head, key channel) from z = W2 act(a) + bias, where a is
//                          the narrow output of a first projection (W2 a may come ready-made from a product):
//                          form 0: sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau);  form 1: exp(-exp(z)).
//   mlb_head_norm_gate     o / sqrt(mean(o^2) + eps) per head, times a weight (one row of DV shared by the heads, or H * DV),
//                          times act(gate) with the gate read from a projection's fp32 output (sigmoid or silu).
//   mlb_lightning_prepare  what enters a recurrence with ONE fixed decay per head: q, k, v = silu of their projection columns
//                          (fp32, partial results summed in split order) and the head's decay written for each of its key channels.
//   mlb_row_norm_gate      o / sqrt(mean(o^2) + eps) over the WHOLE row (all heads together), times a weight of the row's length,
//                          times sigmoid(gate) element by element.
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
    __device__ __forceinline__ float4 at4(long long row, int col) const {      // four columns, 16-byte aligned
        const float* p = base + row * ld + col;
        float4 v = *reinterpret_cast<const float4*>(p);
        for (int k = 1; k < n_partials; ++k) {
            const float4 w = *reinterpret_cast<const float4*>(p + (size_t)k * partial_stride);
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        return v;
    }
    __host__ bool fours(int col) const {
        return !base || (((uintptr_t)base % 16 == 0) && ld % 4 == 0 && col % 4 == 0 && (n_partials <= 1 || partial_stride % 4 == 0));
    }
};

__device__ __forceinline__ float sigmoid(float v) {
    if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}

// log(sigmoid(v)) without overflow on either side
__device__ __forceinline__ float log_sigmoid(float v) { return fminf(v, 0.0f) - log1pf(expf(-fabsf(v))); }

// ------------------------------------------------------------------------------ token shift
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mu, const float* __restrict__ state,
                                   const int* __restrict__ slots, int num_slots, const int* __restrict__ seq_starts,
                                   const int* __restrict__ seq_pos0, const int* __restrict__ token_seq, T* __restrict__ out,
                                   int tokens, int width, int n_mix, int* error_flag) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    const int a = token_seq[t];
    const float now = to_f32(x[i]);
    float before;
    if (t > seq_starts[a]) {
        before = to_f32(x[i - width]);
    } else if (seq_pos0[a] == 0) {
        before = 0.0f;
    } else {
        const int slot = slots[a];
        if (slot < 0 || slot >= num_slots) {
            if (error_flag) atomicExch(error_flag, 3);
            return;
        }
        before = state[(size_t)slot * width + c];
    }
    const float back = before - now;
    for (int s = 0; s < n_mix; ++s)
        out[((size_t)s * tokens + t) * width + c] = from_f32<T>(fmaf(back, mu[(size_t)s * width + c], now));
}

// The same, 16 bytes of a row a thread (eight bf16 or four fp32 channels): widths that are a multiple of that.
template <typename T>
__global__ void token_shift_vec_kernel(const T* __restrict__ x, const float* __restrict__ mu, const float* __restrict__ state,
                                       const int* __restrict__ slots, int num_slots, const int* __restrict__ seq_starts,
                                       const int* __restrict__ seq_pos0, const int* __restrict__ token_seq, T* __restrict__ out,
                                       int tokens, int width, int n_mix, int* error_flag) {
    constexpr int N = 16 / sizeof(T);
    pdl_prologue();
    const int pieces = width / N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * pieces) return;
    const int t = (int)(i / pieces), c = (int)(i % pieces) * N;
    const int a = token_seq[t];
    const size_t at = (size_t)t * width + c;
    float now[N], back[N];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + at);
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < N; ++j) now[j] = to_f32(v[j]);
    }
    if (t > seq_starts[a]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + at - width);
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < N; ++j) back[j] = to_f32(v[j]) - now[j];
    } else if (seq_pos0[a] == 0) {
#pragma unroll
        for (int j = 0; j < N; ++j) back[j] = -now[j];
    } else {
        const int slot = slots[a];
        if (slot < 0 || slot >= num_slots) {
            if (error_flag) atomicExch(error_flag, 3);
            return;
        }
        const float* st = state + (size_t)slot * width + c;
#pragma unroll
        for (int j = 0; j < N; j += 4) {
            const float4 f = *reinterpret_cast<const float4*>(st + j);
            back[j] = f.x - now[j]; back[j + 1] = f.y - now[j + 1]; back[j + 2] = f.z - now[j + 2]; back[j + 3] = f.w - now[j + 3];
        }
    }
    for (int s = 0; s < n_mix; ++s) {
        const float* m = mu + (size_t)s * width + c;
        uint4 raw;
        T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int j = 0; j < N; j += 4) {
            const float4 f = *reinterpret_cast<const float4*>(m + j);
            v[j] = from_f32<T>(fmaf(back[j], f.x, now[j])); v[j + 1] = from_f32<T>(fmaf(back[j + 1], f.y, now[j + 1]));
            v[j + 2] = from_f32<T>(fmaf(back[j + 2], f.z, now[j + 2])); v[j + 3] = from_f32<T>(fmaf(back[j + 3], f.w, now[j + 3]));
        }
        *reinterpret_cast<uint4*>(out + ((size_t)s * tokens + t) * width + c) = raw;
    }
}

template <typename T>
__global__ void token_shift_state_kernel(const T* __restrict__ x, float* __restrict__ state, const int* __restrict__ slots,
                                         int num_slots, const int* __restrict__ seq_starts, int seqs, int width) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)seqs * width) return;
    const int a = (int)(i / width), c = (int)(i % width);
    const int last = seq_starts[a + 1] - 1, slot = slots[a];
    if (last < seq_starts[a] || slot < 0 || slot >= num_slots) return;
    state[(size_t)slot * width + c] = to_f32(x[(size_t)last * width + c]);
}

// ------------------------------------------------------------------------------ what enters the recurrence
struct PrepareParams {
    Columns q, k, v; int q_col, k_col, v_col;      // q, k: H * DK columns each; v: H * DV
    float q_scale;
    Columns narrow; int a_col; int rank; int narrow_act;      // a [rank] (narrow_act 1: tanh of it); used when `pre` has no base
    const float* w2;                               // [H * DK, rank] fp32
    Columns pre;                                   // W2 act(a) ready-made [T, H * DK]
    const float* bias;                             // [H * DK], may be null
    int form; float inv_tau;
    float* q_out; float* k_out; float* v_out; float* decay;   // [T, H * DK] x 2, [T, H * DV], [T, H * DK]
    int T, HK, HV;
};

__global__ void decay_prepare_kernel(PrepareParams p) {
    pdl_prologue();
    const int per_token = 3 * p.HK + p.HV;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.T * per_token) return;
    const long long t = i / per_token;
    int c = (int)(i % per_token);
    if (c < p.HK) { p.q_out[t * p.HK + c] = p.q.at(t, p.q_col + c) * p.q_scale; return; }
    c -= p.HK;
    if (c < p.HK) { p.k_out[t * p.HK + c] = p.k.at(t, p.k_col + c); return; }
    c -= p.HK;
    if (c < p.HV) { p.v_out[t * p.HV + c] = p.v.at(t, p.v_col + c); return; }
    c -= p.HV;
    float z = 0.0f;
    if (p.pre.base) {
        z = p.pre.at(t, c);
    } else {
        const float* w = p.w2 + (size_t)c * p.rank;
        for (int r = 0; r < p.rank; ++r) {
            float a = p.narrow.at(t, p.a_col + r);
            if (p.narrow_act == 1) a = tanhf(a);
            z = fmaf(w[r], a, z);
        }
    }
    if (p.bias) z += p.bias[c];
    p.decay[t * p.HK + c] = p.form == 0 ? expf(log_sigmoid(z) * p.inv_tau) : expf(-expf(z));
}

// The same, four columns a thread (16-byte loads and stores): every block of columns starts and ends on a multiple of four.
__global__ void decay_prepare_x4_kernel(PrepareParams p) {
    pdl_prologue();
    const int per_token = (3 * p.HK + p.HV) / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.T * per_token) return;
    const long long t = i / per_token;
    int c = (int)(i % per_token) * 4;
    if (c < p.HK) {
        float4 q = p.q.at4(t, p.q_col + c);
        q.x *= p.q_scale; q.y *= p.q_scale; q.z *= p.q_scale; q.w *= p.q_scale;
        *reinterpret_cast<float4*>(p.q_out + t * p.HK + c) = q;
        return;
    }
    c -= p.HK;
    if (c < p.HK) { *reinterpret_cast<float4*>(p.k_out + t * p.HK + c) = p.k.at4(t, p.k_col + c); return; }
    c -= p.HK;
    if (c < p.HV) { *reinterpret_cast<float4*>(p.v_out + t * p.HV + c) = p.v.at4(t, p.v_col + c); return; }
    c -= p.HV;
    float z[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (p.pre.base) {
        const float4 f = p.pre.at4(t, c);
        z[0] = f.x; z[1] = f.y; z[2] = f.z; z[3] = f.w;
    } else {
        const float* w = p.w2 + (size_t)c * p.rank;
        for (int r = 0; r < p.rank; ++r) {
            float a = p.narrow.at(t, p.a_col + r);
            if (p.narrow_act == 1) a = tanhf(a);
#pragma unroll
            for (int j = 0; j < 4; ++j) z[j] = fmaf(w[(size_t)j * p.rank + r], a, z[j]);
        }
    }
    if (p.bias) {
        const float4 b = *reinterpret_cast<const float4*>(p.bias + c);
        z[0] += b.x; z[1] += b.y; z[2] += b.z; z[3] += b.w;
    }
    float4 d;
    if (p.form == 0) {
        d.x = expf(log_sigmoid(z[0]) * p.inv_tau); d.y = expf(log_sigmoid(z[1]) * p.inv_tau);
        d.z = expf(log_sigmoid(z[2]) * p.inv_tau); d.w = expf(log_sigmoid(z[3]) * p.inv_tau);
    } else {
        d.x = expf(-expf(z[0])); d.y = expf(-expf(z[1])); d.z = expf(-expf(z[2])); d.w = expf(-expf(z[3]));
    }
    *reinterpret_cast<float4*>(p.decay + t * p.HK + c) = d;
}

// ------------------------------------------------------------------------------ output norm and gate
struct OutputParams {
    const float* o;                          // [T, H * DV]
    const float* weight; int weight_per_head;      // [DV] shared by the heads (0) or [H * DV] (1); null: no weight
    Columns gate; int gate_col; int gate_act;      // gate.base null: no gate; 0 sigmoid, 1 silu
    void* out;                               // [T, H * DV]
    int T, H, DV; float eps;
};

template <typename OutT>
__global__ void __launch_bounds__(WARPS * 32) head_norm_gate_kernel(OutputParams p) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * p.H) return;
    const int t = (int)(item / p.H), h = (int)(item % p.H);
    const float* src = p.o + ((size_t)t * p.H + h) * p.DV;
    float x[PER_LANE];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        x[i] = c < p.DV ? src[c] : 0.0f;
        ss = fmaf(x[i], x[i], ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.DV + p.eps);
    OutT* dst = (OutT*)p.out + ((size_t)t * p.H + h) * p.DV;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c >= p.DV) continue;
        float y = x[i] * inv;
        if (p.weight) y *= p.weight[p.weight_per_head ? h * p.DV + c : c];
        if (p.gate.base) {
            const float g = p.gate.at(t, p.gate_col + h * p.DV + c);
            y *= p.gate_act == 1 ? g * sigmoid(g) : sigmoid(g);
        }
        dst[c] = from_f32<OutT>(y);
    }
}

// The same, four columns a lane (16-byte loads of o and the gate, 8- or 16-byte stores): DV a multiple of four.
template <typename OutT>
__global__ void __launch_bounds__(WARPS * 32) head_norm_gate_x4_kernel(OutputParams p) {
    constexpr int QUADS = MAX_D / 128;
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * p.H) return;
    const int t = (int)(item / p.H), h = (int)(item % p.H);
    const float* src = p.o + ((size_t)t * p.H + h) * p.DV;
    float4 x[QUADS], g[QUADS];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < QUADS; ++i) {
        const int c = 4 * lane + 128 * i;
        x[i] = c < p.DV ? *reinterpret_cast<const float4*>(src + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (p.gate.base && c < p.DV) g[i] = p.gate.at4(t, p.gate_col + h * p.DV + c);
        ss = fmaf(x[i].x, x[i].x, ss); ss = fmaf(x[i].y, x[i].y, ss); ss = fmaf(x[i].z, x[i].z, ss); ss = fmaf(x[i].w, x[i].w, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.DV + p.eps);
    OutT* dst = (OutT*)p.out + ((size_t)t * p.H + h) * p.DV;
#pragma unroll
    for (int i = 0; i < QUADS; ++i) {
        const int c = 4 * lane + 128 * i;
        if (c >= p.DV) continue;
        float y[4] = {x[i].x * inv, x[i].y * inv, x[i].z * inv, x[i].w * inv};
        if (p.weight) {
            const float4 w = *reinterpret_cast<const float4*>(p.weight + (p.weight_per_head ? h * p.DV + c : c));
            y[0] *= w.x; y[1] *= w.y; y[2] *= w.z; y[3] *= w.w;
        }
        if (p.gate.base) {
            const float gs[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) y[j] *= p.gate_act == 1 ? gs[j] * sigmoid(gs[j]) : sigmoid(gs[j]);
        }
        if constexpr (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(dst + c) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
            uint2 raw;
            OutT* v = reinterpret_cast<OutT*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = from_f32<OutT>(y[j]);
            *reinterpret_cast<uint2*>(dst + c) = raw;
        }
    }
}

}  // namespace

MLB_EXPORT int mlb_token_shift(const void* x, int dtype, const float* mu, const float* state, const int* slots, int num_slots,
                               const int* seq_starts, const int* seq_pos0, const int* token_seq, void* out, int tokens, int width,
                               int n_mix, int* error_flag, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || n_mix <= 0 || !x || !mu || !state || !slots || !seq_starts || !seq_pos0 || !token_seq || !out)
        return fail(MLB_INVALID_ARGUMENT, "token_shift: bad operands");
    if (tokens == 0) return MLB_OK;
    const int per = dtype == MLB_BF16 ? 8 : 4;
    const bool vec = width % per == 0 && ((uintptr_t)x | (uintptr_t)out | (uintptr_t)mu | (uintptr_t)state) % 16 == 0;
    if (vec && (dtype == MLB_BF16 || dtype == MLB_F32)) {
        const unsigned vec_blocks = (unsigned)(((long long)tokens * (width / per) + 255) / 256);
        if (dtype == MLB_BF16)
            launch_kernel(token_shift_vec_kernel<__nv_bfloat16>, vec_blocks, 256, 0, stream, (const __nv_bfloat16*)x, mu, state, slots,
                          num_slots, seq_starts, seq_pos0, token_seq, (__nv_bfloat16*)out, tokens, width, n_mix, error_flag);
        else
            launch_kernel(token_shift_vec_kernel<float>, vec_blocks, 256, 0, stream, (const float*)x, mu, state, slots, num_slots,
                          seq_starts, seq_pos0, token_seq, (float*)out, tokens, width, n_mix, error_flag);
        return check_launch("token_shift");
    }
    const unsigned blocks = (unsigned)(((long long)tokens * width + 255) / 256);
    if (dtype == MLB_BF16)
        launch_kernel(token_shift_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, mu, state, slots, num_slots,
                      seq_starts, seq_pos0, token_seq, (__nv_bfloat16*)out, tokens, width, n_mix, error_flag);
    else if (dtype == MLB_F32)
        launch_kernel(token_shift_kernel<float>, blocks, 256, 0, stream, (const float*)x, mu, state, slots, num_slots, seq_starts,
                      seq_pos0, token_seq, (float*)out, tokens, width, n_mix, error_flag);
    else return fail(MLB_INVALID_ARGUMENT, "token_shift: unsupported dtype %d", dtype);
    return check_launch("token_shift");
}

MLB_EXPORT int mlb_token_shift_state(const void* x, int dtype, float* state, const int* slots, int num_slots, const int* seq_starts,
                                     int seqs, int width, cudaStream_t stream) {
    if (seqs < 0 || width <= 0 || !x || !state || !slots || !seq_starts) return fail(MLB_INVALID_ARGUMENT, "token_shift_state: bad operands");
    if (seqs == 0) return MLB_OK;
    const unsigned blocks = (unsigned)(((long long)seqs * width + 255) / 256);
    if (dtype == MLB_BF16)
        launch_kernel(token_shift_state_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, state, slots, num_slots,
                      seq_starts, seqs, width);
    else if (dtype == MLB_F32)
        launch_kernel(token_shift_state_kernel<float>, blocks, 256, 0, stream, (const float*)x, state, slots, num_slots, seq_starts,
                      seqs, width);
    else return fail(MLB_INVALID_ARGUMENT, "token_shift_state: unsupported dtype %d", dtype);
    return check_launch("token_shift_state");
}

MLB_EXPORT int mlb_decay_prepare(const float* q, long long q_ld, int q_partials, long long q_stride, int q_col,
                                 const float* k, long long k_ld, int k_partials, long long k_stride, int k_col,
                                 const float* v, long long v_ld, int v_partials, long long v_stride, int v_col, float q_scale,
                                 const float* narrow, long long n_ld, int n_partials, long long n_stride, int a_col, int rank,
                                 int narrow_act, const float* w2, const float* pre, long long pre_ld, int pre_partials,
                                 long long pre_stride, const float* bias, int form, float tau, float* q_out, float* k_out,
                                 float* v_out, float* decay, int T, int HK, int HV, cudaStream_t stream) {
    if (T < 0 || HK <= 0 || HV <= 0 || !q || !k || !v || !q_out || !k_out || !v_out || !decay || (!pre && (!narrow || !w2 || rank <= 0)))
        return fail(MLB_INVALID_ARGUMENT, "decay_prepare: bad operands");
    if ((form != 0 && form != 1) || (form == 0 && !(tau > 0.0f))) return fail(MLB_INVALID_ARGUMENT, "decay_prepare: form %d, tau %g", form, tau);
    if (T == 0) return MLB_OK;
    auto cols = [](const float* base, long long ld, int n, long long stride) { return Columns{base, ld, n < 1 ? 1 : n, stride}; };
    PrepareParams p{cols(q, q_ld, q_partials, q_stride), cols(k, k_ld, k_partials, k_stride), cols(v, v_ld, v_partials, v_stride),
                    q_col, k_col, v_col, q_scale, cols(narrow, n_ld, n_partials, n_stride), a_col, rank, narrow_act, w2,
                    cols(pre, pre_ld, pre_partials, pre_stride), bias, form, form == 0 ? 1.0f / tau : 0.0f, q_out, k_out, v_out, decay,
                    T, HK, HV};
    const long long n = (long long)T * (3 * HK + HV);
    const bool fours = HK % 4 == 0 && HV % 4 == 0 && p.q.fours(q_col) && p.k.fours(k_col) && p.v.fours(v_col) && p.pre.fours(0) &&
                       ((uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out | (uintptr_t)decay | (uintptr_t)bias) % 16 == 0;
    if (fours) launch_kernel(decay_prepare_x4_kernel, (unsigned)((n / 4 + 255) / 256), 256, 0, stream, p);
    else launch_kernel(decay_prepare_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, p);
    return check_launch("decay_prepare");
}

MLB_EXPORT int mlb_head_norm_gate(const float* o, const float* weight, int weight_per_head, const float* gate, long long gate_ld,
                                  int gate_partials, long long gate_stride, int gate_col, int gate_act, void* out, int out_dtype,
                                  int T, int H, int DV, float eps, cudaStream_t stream) {
    if (T < 0 || H <= 0 || DV <= 0 || DV > MAX_D) return fail(MLB_UNSUPPORTED_SIZE, "head_norm_gate: value width %d (at most %d)", DV, MAX_D);
    if (!o || !out) return fail(MLB_INVALID_ARGUMENT, "head_norm_gate: null operand");
    if (T == 0) return MLB_OK;
    OutputParams p{o, weight, weight_per_head, Columns{gate, gate_ld, gate_partials < 1 ? 1 : gate_partials, gate_stride}, gate_col,
                   gate_act, out, T, H, DV, eps};
    const long long items = (long long)T * H;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const bool fours = DV % 4 == 0 && p.gate.fours(gate_col) && ((uintptr_t)o | (uintptr_t)weight | (uintptr_t)out) % 16 == 0;
    if (fours && out_dtype == MLB_BF16) launch_kernel(head_norm_gate_x4_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else if (fours && out_dtype == MLB_F32) launch_kernel(head_norm_gate_x4_kernel<float>, blocks, WARPS * 32, 0, stream, p);
    else if (out_dtype == MLB_BF16) launch_kernel(head_norm_gate_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else if (out_dtype == MLB_F32) launch_kernel(head_norm_gate_kernel<float>, blocks, WARPS * 32, 0, stream, p);
    else return fail(MLB_INVALID_ARGUMENT, "head_norm_gate: unsupported dtype %d", out_dtype);
    return check_launch("head_norm_gate");
}

namespace {

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }

// one thread per element of q | k | v (HK + HK + HV per token)
__global__ void lightning_prepare_kernel(Columns src, int q_col, int k_col, int v_col, const float* __restrict__ head_decay,
                                         float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                                         float* __restrict__ decay, long long T, int HK, int HV, int DK) {
    pdl_prologue();
    const int per = 2 * HK + HV;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * per) return;
    const long long t = i / per;
    const int c = (int)(i % per);
    if (c < HK) {
        q_out[t * HK + c] = silu_f32(src.at(t, q_col + c));
        decay[t * HK + c] = head_decay[c / DK];
    } else if (c < 2 * HK) {
        k_out[t * HK + c - HK] = silu_f32(src.at(t, k_col + c - HK));
    } else {
        v_out[t * HV + c - 2 * HK] = silu_f32(src.at(t, v_col + c - 2 * HK));
    }
}

// the same, four neighbouring columns a thread (16-byte loads and stores); HK, HV and DK are multiples of 4
__global__ void lightning_prepare_x4_kernel(Columns src, int q_col, int k_col, int v_col, const float* __restrict__ head_decay,
                                            float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                                            float* __restrict__ decay, long long T, int HK, int HV, int DK) {
    pdl_prologue();
    const int per = (2 * HK + HV) / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * per) return;
    const long long t = i / per;
    const int c = (int)(i % per) * 4;
    auto act = [](float4 v) { return make_float4(silu_f32(v.x), silu_f32(v.y), silu_f32(v.z), silu_f32(v.w)); };
    if (c < HK) {
        *reinterpret_cast<float4*>(q_out + t * HK + c) = act(src.at4(t, q_col + c));
        const float d = head_decay[c / DK];
        *reinterpret_cast<float4*>(decay + t * HK + c) = make_float4(d, d, d, d);
    } else if (c < 2 * HK) {
        *reinterpret_cast<float4*>(k_out + t * HK + c - HK) = act(src.at4(t, k_col + c - HK));
    } else {
        *reinterpret_cast<float4*>(v_out + t * HV + c - 2 * HK) = act(src.at4(t, v_col + c - 2 * HK));
    }
}

constexpr int ROW_THREADS = 256;
template <typename OutT>
__global__ void __launch_bounds__(ROW_THREADS)
row_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, Columns gate, int gate_col, OutT* __restrict__ out,
                     int width, float eps) {
    pdl_prologue();
    __shared__ float scratch[32];
    const long long t = blockIdx.x;
    const float* row = o + (size_t)t * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) ss = fmaf(row[c], row[c], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
        float v = row[c] * inv * (weight ? weight[c] : 1.0f);
        if (gate.base) {
            const float g = gate.at(t, gate_col + c);
            v *= g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g));
        }
        out[(size_t)t * width + c] = from_f32<OutT>(v);
    }
}

}  // namespace

MLB_EXPORT int mlb_lightning_prepare(const float* src, long long ld, int n_partials, long long partial_stride, int q_col, int k_col,
                                     int v_col, const float* head_decay, float* q_out, float* k_out, float* v_out, float* decay,
                                     int T, int H, int DK, int DV, cudaStream_t stream) {
    if (T < 0 || H <= 0 || DK <= 0 || DV <= 0 || n_partials < 1 || !src || !head_decay || !q_out || !k_out || !v_out || !decay)
        return fail(MLB_INVALID_ARGUMENT, "lightning_prepare: bad operands");
    if (T == 0) return MLB_OK;
    const long long n = (long long)T * (2LL * H * DK + (long long)H * DV);
    const Columns cols{src, ld, n_partials, partial_stride};
    const bool fours = DK % 4 == 0 && DV % 4 == 0 && cols.fours(q_col) && cols.fours(k_col) && cols.fours(v_col) &&
                       ((uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out | (uintptr_t)decay) % 16 == 0;
    if (fours)
        launch_kernel(lightning_prepare_x4_kernel, (unsigned)((n / 4 + 255) / 256), 256, 0, stream, cols, q_col, k_col, v_col, head_decay,
                      q_out, k_out, v_out, decay, (long long)T, H * DK, H * DV, DK);
    else
        launch_kernel(lightning_prepare_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, cols,
                      q_col, k_col, v_col, head_decay, q_out, k_out, v_out, decay, (long long)T, H * DK, H * DV, DK);
    return check_launch("lightning_prepare");
}

MLB_EXPORT int mlb_row_norm_gate(const float* o, const float* weight, const float* gate, long long gate_ld, int gate_partials,
                                 long long gate_stride, int gate_col, void* out, int out_dtype, int T, int width, float eps,
                                 cudaStream_t stream) {
    if (T < 0 || width <= 0 || !o || !out) return fail(MLB_INVALID_ARGUMENT, "row_norm_gate: bad operands");
    if (T == 0) return MLB_OK;
    const Columns g{gate, gate_ld, gate_partials < 1 ? 1 : gate_partials, gate_stride};
    if (out_dtype == MLB_BF16)
        launch_kernel(row_norm_gate_kernel<__nv_bfloat16>, (unsigned)T, ROW_THREADS, 0, stream, o, weight, g, gate_col, (__nv_bfloat16*)out, width, eps);
    else if (out_dtype == MLB_F32)
        launch_kernel(row_norm_gate_kernel<float>, (unsigned)T, ROW_THREADS, 0, stream, o, weight, g, gate_col, (float*)out, width, eps);
    else return fail(MLB_INVALID_ARGUMENT, "row_norm_gate: unsupported dtype %d", out_dtype);
    return check_launch("row_norm_gate");
}
