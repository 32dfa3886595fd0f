// Gated delta rule with one decay per head and key channel, fp32 throughout.  Per head, with S [DK, DV]:
//
//   S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t
//
//   mlb_delta_prepare   what enters the recurrence besides v: q and k as unit vectors per head (x / sqrt(sum x^2 + 1e-6),
//                       q also times DK^-1/2), beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(W2 a + dt_bias)) with a
//                       the (narrow) output of the first of the decay's two projections; W2 is applied here.
//   mlb_delta_scan      the recurrence over the new tokens of every sequence of the step, from the state in the
//                       sequence's slot ([slots, H, DK, DV] fp32; taken as zero when the sequence starts at position 0)
//                       and back into it.  The columns of S never meet: a CTA owns 16 of them for one (sequence,
//                       head), eight or sixteen lanes share a column's DK rows in registers and meet by shuffles twice a token.
//   mlb_delta_output    o / rms(o) per head * weight * sigmoid(W2g a_g), stored in the compute dtype.
//
// The scan kernel also runs the two simpler recurrences with a decay per key channel (mlb_linear_scan, `rule`):
//   rule 1, decayed sum:   S <- diag(g_t) S + k_t v_t^T;   o_t = S^T q_t
//   rule 2, bonus read:    o_t = (S + diag(u) k_t v_t^T)^T q_t;   then S <- diag(g_t) S + k_t v_t^T      (u [H, DK], fixed)
//
// The order of every addition depends on the token's place in its sequence only, never on how the sequence was cut
// into steps: a token's result is the same bits however it is scheduled.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;
constexpr int PER_LANE = MAX_D / 32;

struct Columns {
    const float* base; long long ld; int n_partials; long long partial_stride;
    __device__ __forceinline__ float at(long long row, int col) const {
        const float* p = base + row * ld + col;
        float v = p[0];
        for (int k = 1; k < n_partials; ++k) v += p[(size_t)k * partial_stride];
        return v;
    }
};

__device__ __forceinline__ float sigmoid(float v) {
    if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}

__device__ __forceinline__ float softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// ------------------------------------------------------------------------------ prepare
struct PrepareParams {
    const float* qkv; long long ld_qkv;      // convolved and activated [T, G*DK | G*DK | H*DV]
    Columns proj; int beta_col, a_col;       // the input projection's fp32 output: beta pre-activations [H], a [a_rank]
    const float* w2;                         // [H * DK, a_rank]; unused when `pre` is given
    Columns pre;                             // W2 a already made by a product [T, H * DK] (base null: made here)
    const float* dt_bias;                    // [H * DK]
    const float* a_log;                      // [H]
    float* qn; float* kn;                    // [T, G * DK]
    float* g;                                // [T, H * DK]
    float* beta;                             // [T, H]
    int T, H, G, DK, a_rank;
};

__global__ void __launch_bounds__(WARPS * 32) delta_prepare_kernel(PrepareParams p) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = 2 * p.G + p.H;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.T * items) return;
    const int t = (int)(item / items), which = (int)(item % items);
    if (which < 2 * p.G) {                   // a head of q or of k: unit vector
        const bool is_q = which < p.G;
        const int head = is_q ? which : which - p.G;
        const float* src = p.qkv + (size_t)t * p.ld_qkv + (is_q ? 0 : p.G * p.DK) + head * p.DK;
        float x[PER_LANE];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int c = lane + 32 * i;
            x[i] = c < p.DK ? src[c] : 0.0f;
            ss = fmaf(x[i], x[i], ss);
        }
        float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
        if (is_q) inv *= 1.0f / sqrtf((float)p.DK);
        float* dst = (is_q ? p.qn : p.kn) + ((size_t)t * p.G + head) * p.DK;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) { const int c = lane + 32 * i; if (c < p.DK) dst[c] = x[i] * inv; }
        return;
    }
    const int h = which - 2 * p.G;
    const float rate = expf(p.a_log[h]);
    for (int c = lane; c < p.DK; c += 32) {
        float pre = 0.0f;
        if (p.pre.base) {
            pre = p.pre.at(t, h * p.DK + c);
        } else {
            const float* w = p.w2 + ((size_t)h * p.DK + c) * p.a_rank;
            for (int r = 0; r < p.a_rank; ++r) pre = fmaf(w[r], p.proj.at(t, p.a_col + r), pre);
        }
        pre += p.dt_bias[h * p.DK + c];
        p.g[((size_t)t * p.H + h) * p.DK + c] = expf(-rate * softplus(pre));
    }
    if (lane == 0) p.beta[(size_t)t * p.H + h] = sigmoid(p.proj.at(t, p.beta_col + h));
}

// ------------------------------------------------------------------------------ the recurrence
struct ScanParams {
    const float* qn; const float* kn;        // [T, G * DK]
    const float* g;                          // [T, H * DK]
    const float* beta;                       // [T, H] (the delta rule only; else unused and may be null)
    const float* bonus;                      // [H, DK] (rule 2 only)
    const float* v; long long ld_v;          // [T, H * DV] (a column block of the convolved rows)
    float* o;                                // [T, H * DV]
    float* state;                            // [slots + 1, H, DK, DV]
    const int* slots; int num_slots;
    const int* seq_starts; const int* seq_pos0;
    int A, H, G, DK, DV;
    int vec;                                 // 1: every staged row starts on 16 bytes and is a multiple of four floats long
    int* error_flag;
};

constexpr int SCAN_COLS = 16;            // columns of S a CTA owns unless the kernel is told otherwise (COLS); its threads: COLS * LANES

__device__ __forceinline__ void copy_async_f32(float* to_shared, const float* from, bool real) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(to_shared);
    const int bytes = real ? 4 : 0;                            // 0: the four bytes are filled with zeros
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(from), "r"(bytes) : "memory");
}

__device__ __forceinline__ void copy_async_f32x4(float* to_shared, const float* from, bool real) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(to_shared);
    const int bytes = real ? 16 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(from), "r"(bytes) : "memory");
}

// LANES lanes share a column; ROWS: rows of the column that one lane keeps (DK <= LANES * ROWS, ROWS a multiple of 4): lane
// `part` owns rows 4 LANES j + 4 part + (0..3), so that the lanes of a column read consecutive 16-byte pieces of q, k and g.
// Sixteen lanes a column give an SM eight warps instead of four for the same columns: a token's chain of dependent
// instructions is what the kernel waits for, and two warps a scheduler fill each other's gaps.
// CHUNK: tokens whose q, k, g, v and beta are staged in shared memory at a time; the next chunk is copied there
// asynchronously (cp.async, zero fill for padding) while the present one is computed, so the recurrence never waits for
// global memory inside a chunk.
constexpr int RULE_DELTA = 0, RULE_DECAYED_SUM = 1, RULE_BONUS_READ = 2;

template <int LANES, int ROWS, int CHUNK, int RULE, int COLS = SCAN_COLS>
__global__ void __launch_bounds__(COLS * LANES) delta_scan_kernel(ScanParams p) {
    pdl_prologue();
    constexpr int SCAN_LANES = LANES, SCAN_THREADS = COLS * LANES;
    constexpr int DKP = SCAN_LANES * ROWS;                    // padded key width
    constexpr int PER_TOKEN = 3 * DKP + COLS + 4;        // q | k | g | v of this CTA's columns | beta and three unused
    constexpr int STAGED = CHUNK * PER_TOKEN;
    __shared__ __align__(16) float stage_s[2][STAGED];
    const int col_blocks = (p.DV + COLS - 1) / COLS;
    const int cb = blockIdx.x % col_blocks, h = (blockIdx.x / col_blocks) % p.H, a = blockIdx.x / (col_blocks * p.H);
    const int part = threadIdx.x & (SCAN_LANES - 1);
    const int local_col = threadIdx.x / SCAN_LANES;
    const int col = cb * COLS + local_col;
    const bool col_ok = col < p.DV;
    const int start = p.seq_starts[a], n = p.seq_starts[a + 1] - start;
    const int slot = p.slots[a];
    if (slot < 0 || slot >= p.num_slots) {
        if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 3);
        return;
    }
    const int kvh = h / (p.H / p.G);
    auto row_of = [&](int i) { return (i >> 2) * (4 * LANES) + part * 4 + (i & 3); };
    float S[ROWS];
    float* st = p.state + (((size_t)slot * p.H + h) * p.DK) * p.DV;
    const bool fresh = p.seq_pos0[a] == 0;
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
        S[i] = (!fresh && col_ok && row_of(i) < p.DK) ? st[(size_t)row_of(i) * p.DV + col] : 0.0f;
    float U[RULE == RULE_BONUS_READ ? ROWS : 1];
    if (RULE == RULE_BONUS_READ) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) U[i] = row_of(i) < p.DK ? p.bonus[(size_t)h * p.DK + row_of(i)] : 0.0f;
    }

    const float* const q_base = p.qn + ((size_t)start * p.G + kvh) * p.DK;
    const float* const k_base = p.kn + ((size_t)start * p.G + kvh) * p.DK;
    const float* const g_base = p.g + ((size_t)start * p.H + h) * p.DK;
    const float* const v_base = p.v + (size_t)start * p.ld_v + (size_t)h * p.DV;
    const float* const b_base = p.beta ? p.beta + (size_t)start * p.H + h : g_base;     // without beta: any readable address, the value is unused
    const size_t qk_pitch = (size_t)p.G * p.DK, g_pitch = (size_t)p.H * p.DK;
    // the chunk that begins at token `first` into staging buffer `buf`; padding (rows beyond DK, columns beyond DV,
    // tokens beyond the sequence's) becomes zero: a zero k and q keep such rows of S at zero whatever g is
    auto stage = [&](int first, int buf) {
        if (p.vec) {                             // every row a multiple of four floats and 16-byte aligned: four at a time
            constexpr int UNITS = 3 * DKP / 4 + COLS / 4 + 1;
            for (int e = threadIdx.x; e < CHUNK * UNITS; e += SCAN_THREADS) {
                const int tok = e / UNITS, u = e % UNITS;
                const bool live = first + tok < n;
                const size_t t = live ? (size_t)(first + tok) : 0;
                float* to = &stage_s[buf][tok * PER_TOKEN];
                if (u < 3 * DKP / 4) {
                    const int which = u / (DKP / 4), c = (u % (DKP / 4)) * 4;
                    const bool real = c < p.DK;
                    const float* at = (which == 0 ? q_base + t * qk_pitch : (which == 1 ? k_base + t * qk_pitch : g_base + t * g_pitch)) + (real ? c : 0);
                    copy_async_f32x4(to + which * DKP + c, at, live && real);
                } else if (u < UNITS - 1) {
                    const int c = (u - 3 * DKP / 4) * 4, vc = cb * COLS + c;
                    const bool real = vc < p.DV;
                    copy_async_f32x4(to + 3 * DKP + c, v_base + t * p.ld_v + (real ? vc : 0), live && real);
                } else {
                    copy_async_f32(to + 3 * DKP + COLS, b_base + t * p.H, live);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        for (int e = threadIdx.x; e < STAGED; e += SCAN_THREADS) {
            const int tok = e / PER_TOKEN, w = e % PER_TOKEN;
            const bool live = first + tok < n;
            const size_t t = live ? (size_t)(first + tok) : 0;
            const int which = w / DKP, c = w % DKP;
            const int vc = cb * COLS + (w - 3 * DKP);
            const float* at;
            bool real;
            if (which == 0) { real = c < p.DK; at = q_base + t * qk_pitch + (real ? c : 0); }
            else if (which == 1) { real = c < p.DK; at = k_base + t * qk_pitch + (real ? c : 0); }
            else if (which == 2) { real = c < p.DK; at = g_base + t * g_pitch + (real ? c : 0); }
            else if (w < 3 * DKP + COLS) { real = vc < p.DV; at = v_base + t * p.ld_v + (real ? vc : 0); }
            else { real = w == 3 * DKP + COLS; at = b_base + t * p.H; }
            copy_async_f32(&stage_s[buf][e], at, live && real);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    for (int first = 0, buf = 0; first < n; first += CHUNK, buf ^= 1) {
        if (first + CHUNK < n) stage(first + CHUNK, buf ^ 1);
        const int count = min(CHUNK, n - first);
        float* const o_at = p.o + ((size_t)start + first) * ((size_t)p.H * p.DV) + (size_t)h * p.DV + col;
        // `lone`: the lanes of a column meet for this token alone and its o is stored; else the lane's share of o is handed
        // back and the lanes meet once for a group of tokens (below)
        auto token = [&](int tok, bool lone) -> float {
            const float* row = stage_s[buf] + tok * PER_TOKEN;
            const float4* qs = reinterpret_cast<const float4*>(row) + part;
            const float4* ks = reinterpret_cast<const float4*>(row + DKP) + part;
            const float4* gs = reinterpret_cast<const float4*>(row + 2 * DKP) + part;
            const float v = row[3 * DKP + local_col], beta = row[3 * DKP + COLS];
            float4 kk[ROWS / 4];
            if (RULE != RULE_DELTA) {
                // S <- diag(g) S + k v^T with the read-out S^T q behind it (decayed sum), or in front of it with the
                // bonus u on the present token's own k v^T (bonus read); one meeting of the lanes a token
                float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
                for (int j = 0; j < ROWS / 4; ++j) {
                    const float4 gg = gs[j * LANES], qq = qs[j * LANES];
                    kk[j] = ks[j * LANES];
                    const float kv0 = kk[j].x * v, kv1 = kk[j].y * v, kv2 = kk[j].z * v, kv3 = kk[j].w * v;
                    if (RULE == RULE_BONUS_READ) {
                        o0 = fmaf(fmaf(U[4 * j + 0], kv0, S[4 * j + 0]), qq.x, o0); o1 = fmaf(fmaf(U[4 * j + 1], kv1, S[4 * j + 1]), qq.y, o1);
                        o2 = fmaf(fmaf(U[4 * j + 2], kv2, S[4 * j + 2]), qq.z, o2); o3 = fmaf(fmaf(U[4 * j + 3], kv3, S[4 * j + 3]), qq.w, o3);
                    }
                    S[4 * j + 0] = fmaf(S[4 * j + 0], gg.x, kv0); S[4 * j + 1] = fmaf(S[4 * j + 1], gg.y, kv1);
                    S[4 * j + 2] = fmaf(S[4 * j + 2], gg.z, kv2); S[4 * j + 3] = fmaf(S[4 * j + 3], gg.w, kv3);
                    if (RULE == RULE_DECAYED_SUM) {
                        o0 = fmaf(S[4 * j + 0], qq.x, o0); o1 = fmaf(S[4 * j + 1], qq.y, o1);
                        o2 = fmaf(S[4 * j + 2], qq.z, o2); o3 = fmaf(S[4 * j + 3], qq.w, o3);
                    }
                }
                float out = (o0 + o1) + (o2 + o3);
                if (!lone) return out;
#pragma unroll
                for (int off = LANES / 2; off >= 1; off >>= 1) out += __shfl_xor_sync(0xffffffffu, out, off);
                if (part == 0 && col_ok) o_at[(size_t)tok * ((size_t)p.H * p.DV)] = out;
                return 0.0f;
            }
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;          // four chains instead of one (always the same four)
#pragma unroll
            for (int j = 0; j < ROWS / 4; ++j) {
                const float4 gg = gs[j * LANES];
                kk[j] = ks[j * LANES];
                S[4 * j + 0] *= gg.x; S[4 * j + 1] *= gg.y; S[4 * j + 2] *= gg.z; S[4 * j + 3] *= gg.w;
                d0 = fmaf(S[4 * j + 0], kk[j].x, d0); d1 = fmaf(S[4 * j + 1], kk[j].y, d1);
                d2 = fmaf(S[4 * j + 2], kk[j].z, d2); d3 = fmaf(S[4 * j + 3], kk[j].w, d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (LANES == 16) dot += __shfl_xor_sync(0xffffffffu, dot, 8);
            const float u = beta * (v - dot);
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
            for (int j = 0; j < ROWS / 4; ++j) {
                const float4 qq = qs[j * LANES];
                S[4 * j + 0] = fmaf(kk[j].x, u, S[4 * j + 0]); S[4 * j + 1] = fmaf(kk[j].y, u, S[4 * j + 1]);
                S[4 * j + 2] = fmaf(kk[j].z, u, S[4 * j + 2]); S[4 * j + 3] = fmaf(kk[j].w, u, S[4 * j + 3]);
                o0 = fmaf(S[4 * j + 0], qq.x, o0); o1 = fmaf(S[4 * j + 1], qq.y, o1);
                o2 = fmaf(S[4 * j + 2], qq.z, o2); o3 = fmaf(S[4 * j + 3], qq.w, o3);
            }
            float out = (o0 + o1) + (o2 + o3);
            out += __shfl_xor_sync(0xffffffffu, out, 1);
            out += __shfl_xor_sync(0xffffffffu, out, 2);
            out += __shfl_xor_sync(0xffffffffu, out, 4);
            if (LANES == 16) out += __shfl_xor_sync(0xffffffffu, out, 8);
            if (part == 0 && col_ok) o_at[(size_t)tok * ((size_t)p.H * p.DV)] = out;
            return 0.0f;
        };
        if (count == CHUNK && RULE != RULE_DELTA) {
            // A whole chunk of a rule whose read-out nothing waits for: the lanes of a column keep their shares of o for a
            // group of GROUP tokens and meet once for all of them.  A stage at distance `off` halves what a lane carries:
            // it keeps the half of the group's tokens that its own bit `off` names and adds the partner's share of those,
            // so that after the last stage lane `part` holds the whole o of token `part` of the group: GROUP - 1 shuffles
            // for GROUP tokens instead of log2(LANES) each.  Every sum is the one the lone form makes (the same pairs at the
            // same distances, largest first), so both forms give the same bits.
            constexpr int GROUP = CHUNK < LANES ? CHUNK : LANES;
#pragma unroll
            for (int g0 = 0; g0 < CHUNK; g0 += GROUP) {
                float share[GROUP];
#pragma unroll
                for (int i = 0; i < GROUP; ++i) share[i] = token(g0 + i, false);
#pragma unroll
                for (int off = LANES / 2; off >= GROUP; off >>= 1) {
#pragma unroll
                    for (int i = 0; i < GROUP; ++i) share[i] += __shfl_xor_sync(0xffffffffu, share[i], off);
                }
#pragma unroll
                for (int off = GROUP / 2; off >= 1; off >>= 1) {
                    const bool upper = (part & off) != 0;
#pragma unroll
                    for (int i = 0; i < off; ++i) {
                        const float keep = upper ? share[i + off] : share[i];
                        const float send = upper ? share[i] : share[i + off];
                        share[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
                if (part < GROUP && col_ok) o_at[(size_t)(g0 + part) * ((size_t)p.H * p.DV)] = share[0];
            }
        } else if (count == CHUNK) {     // a whole chunk: unrolled, so that a token's read-out runs beside the next token's update
#pragma unroll
            for (int tok = 0; tok < CHUNK; ++tok) token(tok, true);
        } else {
            for (int tok = 0; tok < count; ++tok) token(tok, true);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
        if (col_ok && row_of(i) < p.DK) st[(size_t)row_of(i) * p.DV + col] = S[i];
}

// ------------------------------------------------------------------------------ output norm and gate
struct OutputParams {
    const float* o;                          // [T, H * DV]
    const float* weight;                     // [DV]
    Columns proj; int g_col;                 // the narrow output of the gate's first projection [g_rank]
    const float* w2;                         // [H * DV, g_rank]; unused when `pre` is given
    Columns pre;                             // W2g a_g already made by a product [T, H * DV] (base null: made here)
    void* out;                               // [T, H * DV]
    int T, H, DV, g_rank; float eps;
};

template <typename OutT>
__global__ void __launch_bounds__(WARPS * 32) delta_output_kernel(OutputParams p) {
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
        float pre = 0.0f;
        if (p.pre.base) {
            pre = p.pre.at(t, h * p.DV + c);
        } else {
            const float* w = p.w2 + ((size_t)h * p.DV + c) * p.g_rank;
            for (int r = 0; r < p.g_rank; ++r) pre = fmaf(w[r], p.proj.at(t, p.g_col + r), pre);
        }
        dst[c] = from_f32<OutT>(x[i] * inv * p.weight[c] * sigmoid(pre));
    }
}

// out[t, c] = src[t, col0 + c] (partial results summed in split order), stored in the compute dtype: the narrow output of
// a first projection made ready for the second one (`activation` 1: its tanh).
template <typename OutT>
__global__ void take_columns_kernel(Columns src, int col0, int n, int T, OutT* out, int activation) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T * n) return;
    const float v = src.at(i / n, col0 + (int)(i % n));
    out[i] = from_f32<OutT>(activation == 1 ? tanhf(v) : v);
}

}  // namespace

MLB_EXPORT int mlb_take_columns(const float* src, long long ld, int n_partials, long long partial_stride, int col0, int n, int T,
                                void* out, int out_dtype, int activation, cudaStream_t stream) {
    if (!src || !out || n <= 0 || T < 0 || activation < 0 || activation > 1) return fail(MLB_INVALID_ARGUMENT, "take_columns: bad operands");
    if (T == 0) return MLB_OK;
    Columns c{src, ld, n_partials < 1 ? 1 : n_partials, partial_stride};
    const unsigned blocks = (unsigned)(((long long)T * n + 255) / 256);
    if (out_dtype == MLB_BF16) launch_kernel(take_columns_kernel<__nv_bfloat16>, blocks, 256, 0, stream, c, col0, n, T, (__nv_bfloat16*)out, activation);
    else launch_kernel(take_columns_kernel<float>, blocks, 256, 0, stream, c, col0, n, T, (float*)out, activation);
    return check_launch("take_columns");
}

MLB_EXPORT int mlb_delta_prepare(const float* qkv, long long ld_qkv, const float* proj, long long ld_proj, int n_partials,
                                 long long partial_stride, int beta_col, int a_col, const float* w2, const float* pre, long long ld_pre,
                                 int pre_partials, long long pre_partial_stride, const float* dt_bias,
                                 const float* a_log, float* qn, float* kn, float* g, float* beta, int T, int H, int G, int DK,
                                 int a_rank, cudaStream_t stream) {
    if (T < 0 || H <= 0 || G <= 0 || H % G || DK <= 0 || DK > MAX_D || a_rank <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "delta_prepare: heads %d/%d, key width %d (at most %d), rank %d", H, G, DK, MAX_D, a_rank);
    if (!qkv || !proj || (!w2 && !pre) || !dt_bias || !a_log || !qn || !kn || !g || !beta) return fail(MLB_INVALID_ARGUMENT, "delta_prepare: null operand");
    if (T == 0) return MLB_OK;
    PrepareParams p{qkv, ld_qkv, Columns{proj, ld_proj, n_partials < 1 ? 1 : n_partials, partial_stride}, beta_col, a_col, w2,
                    Columns{pre, ld_pre, pre_partials < 1 ? 1 : pre_partials, pre_partial_stride}, dt_bias, a_log, qn, kn, g, beta, T, H, G, DK, a_rank};
    const long long items = (long long)T * (2 * G + H);
    launch_kernel(delta_prepare_kernel, (unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, stream, p);
    return check_launch("delta_prepare");
}

namespace {

template <int RULE>
int launch_scan(const float* qn, const float* kn, const float* g, const float* beta, const float* bonus, const float* v, long long ld_v,
                float* o, float* state, const int* slots, int num_slots, const int* seq_starts, const int* seq_pos0,
                int A, int H, int G, int DK, int DV, int* error_flag, cudaStream_t stream) {
    if (A < 0 || H <= 0 || G <= 0 || H % G || DK <= 0 || DK > MAX_D || DV <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "scan: heads %d/%d, widths %d (at most %d) / %d", H, G, DK, MAX_D, DV);
    if (!qn || !kn || !g || (RULE == RULE_DELTA && !beta) || (RULE == RULE_BONUS_READ && !bonus) || !v || !o || !state || !slots ||
        !seq_starts || !seq_pos0)
        return fail(MLB_INVALID_ARGUMENT, "scan: null operand");
    if (A == 0) return MLB_OK;
    const bool aligned = ((uintptr_t)qn | (uintptr_t)kn | (uintptr_t)g | (uintptr_t)v) % 16 == 0;
    const int vec = aligned && DK % 4 == 0 && DV % 4 == 0 && ld_v % 4 == 0;
    ScanParams p{qn, kn, g, beta, bonus, v, ld_v, o, state, slots, num_slots, seq_starts, seq_pos0, A, H, G, DK, DV, vec, error_flag};
    // A handful of long-running CTAs (a prompt portion: one CTA walks all its tokens) must be spread one to an SM.  Started
    // early behind a predecessor that still fills the SMs, they land wherever a slot falls free, several on one SM, and
    // the slowest SM decides: such a launch waits for its predecessor the plain way.  Many short CTAs (decoding) start early.
    auto go = [&](auto kernel, int lanes, int cols) {
        const unsigned blocks = (unsigned)((long long)A * H * ((DV + cols - 1) / cols));
        const bool early = blocks > 2u * (unsigned)sm_count();
        if (early) launch_kernel(kernel, blocks, cols * lanes, 0, stream, p);
        else kernel<<<blocks, cols * lanes, 0, stream>>>(p);
    };
    if (DK <= 32) go(delta_scan_kernel<8, 4, 16, RULE>, 8, SCAN_COLS);
    else if (DK <= 64) go(delta_scan_kernel<16, 4, 16, RULE>, 16, SCAN_COLS);
    else if (DK <= 128) go(delta_scan_kernel<16, 8, 8, RULE>, 16, SCAN_COLS);
    else go(delta_scan_kernel<16, 16, 4, RULE>, 16, SCAN_COLS);
    return check_launch("scan");
}

}  // namespace

MLB_EXPORT int mlb_delta_scan(const float* qn, const float* kn, const float* g, const float* beta, const float* v, long long ld_v,
                              float* o, float* state, const int* slots, int num_slots, const int* seq_starts, const int* seq_pos0,
                              int A, int H, int G, int DK, int DV, int* error_flag, cudaStream_t stream) {
    return launch_scan<RULE_DELTA>(qn, kn, g, beta, nullptr, v, ld_v, o, state, slots, num_slots, seq_starts, seq_pos0, A, H, G, DK, DV,
                                   error_flag, stream);
}

// rule 1: S <- diag(g) S + k v^T, o = S^T q;   rule 2: o = (S + diag(bonus) k v^T)^T q, then S <- diag(g) S + k v^T.
// q, k [T, G * DK], g [T, H * DK], bonus [H, DK] (rule 2), v rows of pitch ld_v, o [T, H * DV], state [slots, H, DK, DV].
MLB_EXPORT int mlb_linear_scan(int rule, const float* q, const float* k, const float* g, const float* bonus, const float* v,
                               long long ld_v, float* o, float* state, const int* slots, int num_slots, const int* seq_starts,
                               const int* seq_pos0, int A, int H, int G, int DK, int DV, int* error_flag, cudaStream_t stream) {
    if (rule == RULE_DECAYED_SUM)
        return launch_scan<RULE_DECAYED_SUM>(q, k, g, nullptr, nullptr, v, ld_v, o, state, slots, num_slots, seq_starts, seq_pos0, A, H, G,
                                             DK, DV, error_flag, stream);
    if (rule == RULE_BONUS_READ)
        return launch_scan<RULE_BONUS_READ>(q, k, g, nullptr, bonus, v, ld_v, o, state, slots, num_slots, seq_starts, seq_pos0, A, H, G,
                                            DK, DV, error_flag, stream);
    return fail(MLB_INVALID_ARGUMENT, "linear_scan: unknown rule %d", rule);
}

MLB_EXPORT int mlb_delta_output(const float* o, const float* weight, const float* proj, long long ld_proj, int n_partials,
                                long long partial_stride, int g_col, const float* w2, const float* pre, long long ld_pre,
                                int pre_partials, long long pre_partial_stride, void* out, int out_dtype, int T, int H,
                                int DV, int g_rank, float eps, cudaStream_t stream) {
    if (T < 0 || H <= 0 || DV <= 0 || DV > MAX_D || g_rank <= 0)
        return fail(MLB_UNSUPPORTED_SIZE, "delta_output: value width %d (at most %d), rank %d", DV, MAX_D, g_rank);
    if (!o || !weight || !proj || (!w2 && !pre) || !out) return fail(MLB_INVALID_ARGUMENT, "delta_output: null operand");
    if (T == 0) return MLB_OK;
    OutputParams p{o, weight, Columns{proj, ld_proj, n_partials < 1 ? 1 : n_partials, partial_stride}, g_col, w2,
                   Columns{pre, ld_pre, pre_partials < 1 ? 1 : pre_partials, pre_partial_stride}, out, T, H, DV, g_rank, eps};
    const long long items = (long long)T * H;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (out_dtype == MLB_BF16) launch_kernel(delta_output_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else launch_kernel(delta_output_kernel<float>, blocks, WARPS * 32, 0, stream, p);
    return check_launch("delta_output");
}
