// Mixers that keep a fixed-size state per sequence instead of keys and values:
//
//   * token shift: every stream s of a mixer reads h_t + (h_(t-1) - h_t) * mu_s, where h_(t-1)
//     is the row before in the same sequence or, for a step's first token, the row that the
//     sequence's state holds (zeros at the start of a sequence);
//   * the linear recurrence over a matrix-valued state S (key channel x value channel) per head,
//         o_t = (diag(a_t) S_(t-1) + diag(b) k_t v_t^T)^T q_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T,
//     in its two uses: with a = 1 and a bonus b = u for the current token (output before the
//     decay: the "wkv" form), and with a = w, b = 1 (output after the update: the gated form in
//     which the forget gate f also scales what is written, k = 1 - f);
//   * the per-head unit norm of the recurrence's output, times a weight, times an optional gate.
//
// The state lives in 32-bit floats in the engine's per-sequence state area and is carried from
// step to step; a sequence's tokens are walked in order by one CTA per (sequence, head), thread j
// owning column j of S in registers, so the result does not depend on how the tokens were cut into
// steps or on what else is in the batch.  Decays, gates, exponentials and the state are 32-bit.
#include "common.cuh"

// ------------------------------------------------------------ token shift
// out[s][t][:] = h[t] + (prev - h[t]) * mu[s], s < n_mix.  Rows of sequence -1 are skipped.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state, size_t state_stride, VecRef mu, int n_mix,
                   T* __restrict__ out, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                   const int* __restrict__ seq_slots, int n_rows, int d) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int seq = tok_seq[t];
    int first = 0, slot = 0;
    if (seq >= 0) { first = seq_start[seq]; slot = seq_slots[seq]; }
    pdl_wait();
    if (seq < 0) return;
    const T* hr = h + (size_t)t * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float hv = to_f32(hr[c]);
        const float pv = (t == first) ? state[(size_t)slot * state_stride + c] : to_f32(hr[c - d]);
        const float diff = pv - hv;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * n_rows + t) * d + c] = from_f32<T>(hv + diff * mu.at(s * d + c));
    }
}

extern "C" int odin_token_shift(const void* h, int dtype, const float* state, long long state_stride, const void* mu,
                                int mu_dtype, int n_mix, void* out, const int* tok_seq, const int* seq_start,
                                const int* seq_slots, int n_rows, int d, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0 || n_mix <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef mv{mu, mu_dtype == ODIN_BF16};
    if (dtype == ODIN_BF16)
        odin_launch(token_shift_kernel<bf16>, dim3(n_rows), dim3(256), 0, s, (const bf16*)h, state, (size_t)state_stride,
                    mv, n_mix, (bf16*)out, tok_seq, seq_start, seq_slots, n_rows, d);
    else if (dtype == ODIN_F32)
        odin_launch(token_shift_kernel<float>, dim3(n_rows), dim3(256), 0, s, (const float*)h, state, (size_t)state_stride,
                    mv, n_mix, (float*)out, tok_seq, seq_start, seq_slots, n_rows, d);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ the recurrence
#define REC_BONUS 0   // o = (S + diag(u) k v^T)^T r, then S = diag(w) S + k v^T, w = exp(-exp(raw + w0))
#define REC_GATED 1   // f = l + (1 - l) sigmoid(raw + b); S = diag(f) S + (1 - f) v^T; o = S^T silu(q)
#define REC_TOKENS 8  // tokens whose q, k, w are staged in shared memory together
#define REC_MAX_DK 256

struct RecParams {
    const float* q; long long q_stride;   // [rows, H*dk] projections (32-bit), row strides in elements
    const float* k; long long k_stride;   // REC_BONUS only
    const float* g; long long g_stride;   // the raw decay / forget gate
    const float* v; long long v_stride;   // [rows, H*dv]
    VecRef c0, c1;                        // per (head, key channel): REC_BONUS w0 and u; REC_GATED bias and lower bound
    float* o; long long o_stride;         // [rows, H*dv]
    float* state; long long state_stride; // per slot: [H][dk][dv] floats
    const int* seq_start; const int* seq_slots;
    int H, dk, dv;
    // the token shift's memory: after the step the sequence's last row of h goes to its state
    const void* shift_src; int shift_is_bf16; float* shift_state; long long shift_stride; int width;
};

template <int DK, int MODE>
__global__ void __launch_bounds__(256)
linear_recurrence_kernel(RecParams p) {
    constexpr int NK = DK > 0 ? DK : REC_MAX_DK;
    __shared__ float sq[REC_TOKENS][NK], sk[REC_TOKENS][NK], sw[REC_TOKENS][NK];
    pdl_trigger();
    const int b = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int dk = DK > 0 ? DK : p.dk;
    const int row0 = p.seq_start[b], row1 = p.seq_start[b + 1];
    const int slot = p.seq_slots[b];
    pdl_wait();
    if (row1 <= row0) return;  // an empty (padding) sequence owns no state
    const bool owns = j < p.dv;
    float S[NK];
    float* st = p.state + (size_t)slot * p.state_stride + (size_t)head * dk * p.dv + j;
    if (owns) {
#pragma unroll
        for (int i = 0; i < NK; ++i)
            if (i < dk) S[i] = st[(size_t)i * p.dv];
    }
    const int hc = head * dk;
    for (int t0 = row0; t0 < row1; t0 += REC_TOKENS) {
        const int nt = min(REC_TOKENS, row1 - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) {
            const int u = e / dk, i = e % dk;
            const size_t r = (size_t)(t0 + u);
            const float raw = p.g[r * p.g_stride + hc + i];
            const float qv = p.q[r * p.q_stride + hc + i];
            if (MODE == REC_BONUS) {
                sq[u][i] = qv;
                sk[u][i] = p.k[r * p.k_stride + hc + i];
                sw[u][i] = expf(-expf(raw + p.c0.at(hc + i)));
            } else {
                const float l = p.c1.at(hc + i);
                const float f = l + (1.0f - l) * (1.0f / (1.0f + expf(-(raw + p.c0.at(hc + i)))));
                sq[u][i] = qv / (1.0f + expf(-qv));
                sk[u][i] = 1.0f - f;
                sw[u][i] = f;
            }
        }
        __syncthreads();
        if (owns) {
            for (int u = 0; u < nt; ++u) {
                const size_t r = (size_t)(t0 + u);
                const float vj = p.v[r * p.v_stride + (size_t)head * p.dv + j];
                float acc = 0.f;
                if (MODE == REC_BONUS) {
#pragma unroll
                    for (int i = 0; i < NK; ++i) {
                        if (i < dk) {
                            const float kv = sk[u][i] * vj;
                            acc = fmaf(sq[u][i], fmaf(p.c1.at(hc + i), kv, S[i]), acc);
                            S[i] = fmaf(sw[u][i], S[i], kv);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NK; ++i) {
                        if (i < dk) {
                            S[i] = fmaf(sw[u][i], S[i], sk[u][i] * vj);
                            acc = fmaf(sq[u][i], S[i], acc);
                        }
                    }
                }
                p.o[r * p.o_stride + (size_t)head * p.dv + j] = acc;
            }
        }
    }
    if (owns) {
#pragma unroll
        for (int i = 0; i < NK; ++i)
            if (i < dk) st[(size_t)i * p.dv] = S[i];
    }
    if (head == 0 && p.shift_src != nullptr) {
        float* dst = p.shift_state + (size_t)slot * p.shift_stride;
        const size_t last = (size_t)(row1 - 1) * p.width;
        for (int c = threadIdx.x; c < p.width; c += blockDim.x)
            dst[c] = p.shift_is_bf16 ? __bfloat162float(((const bf16*)p.shift_src)[last + c]) : ((const float*)p.shift_src)[last + c];
    }
}

extern "C" int odin_linear_recurrence(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                                      const float* g, long long g_stride, const float* v, long long v_stride,
                                      const void* c0, const void* c1, int c_dtype, float* o, long long o_stride,
                                      float* state, long long state_stride, const int* seq_start, const int* seq_slots,
                                      int n_seqs, int H, int dk, int dv, const void* shift_src, int shift_dtype,
                                      float* shift_state, long long shift_stride, int width, void* stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || dk <= 0 || dk > REC_MAX_DK || dv <= 0 || dv > 256 || H > 65535) return ODIN_ERR_UNSUPPORTED;
    if (mode != REC_BONUS && mode != REC_GATED) return ODIN_ERR_BAD_ARG;
    RecParams p;
    p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.g = g; p.g_stride = g_stride;
    p.v = v; p.v_stride = v_stride;
    p.c0 = VecRef{c0, c_dtype == ODIN_BF16}; p.c1 = VecRef{c1, c_dtype == ODIN_BF16};
    p.o = o; p.o_stride = o_stride; p.state = state; p.state_stride = state_stride;
    p.seq_start = seq_start; p.seq_slots = seq_slots; p.H = H; p.dk = dk; p.dv = dv;
    p.shift_src = shift_src; p.shift_is_bf16 = shift_dtype == ODIN_BF16; p.shift_state = shift_state;
    p.shift_stride = shift_stride; p.width = width;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = (dv + 31) / 32 * 32;
    dim3 grid(n_seqs, H);
#define GO(DK)                                                                                                  \
    do {                                                                                                        \
        if (mode == REC_BONUS) odin_launch(linear_recurrence_kernel<DK, REC_BONUS>, grid, dim3(threads), 0, s, p);  \
        else odin_launch(linear_recurrence_kernel<DK, REC_GATED>, grid, dim3(threads), 0, s, p);                \
    } while (0)
    switch (dk) {  // the usual sizes keep the state column in registers; any other size up to 256 runs the general kernel
        case 16: GO(16); break;
        case 32: GO(32); break;
        case 48: GO(48); break;
        case 64: GO(64); break;
        case 96: GO(96); break;
        case 128: GO(128); break;
        default: GO(0); break;
    }
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ per-head unit norm, weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[h * w_head_stride + :] * silu(gate[t, h, :])
// One warp per (token, head); the gate is optional.
template <typename TO>
__global__ void __launch_bounds__(128)
head_unit_scale_kernel(const float* __restrict__ o, const VecRef w, int w_head_stride, const float* __restrict__ gate,
                       long long gate_stride, float eps, TO* __restrict__ out, int T, int H, int dv) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
    ss = warp_sum(ss);
    ss /= (float)dv;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    TO* dst = out + ((size_t)t * H + h) * dv;
    for (int c = lane; c < dv; c += 32) {
        float y = w.at(h * w_head_stride + c) * (rs * src[c]);
        if (gate != nullptr) {
            const float z = gate[(size_t)t * gate_stride + (size_t)h * dv + c];
            y *= z / (1.0f + expf(-z));
        }
        dst[c] = from_f32<TO>(y);
    }
}

extern "C" int odin_head_unit_scale(const float* o, const void* w, int w_dtype, int w_head_stride, const float* gate,
                                    long long gate_stride, float eps, void* out, int out_dtype, int T, int H, int dv,
                                    void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long blocks = ((long long)T * H + 3) / 4;
    if (blocks > 2147483647LL) return ODIN_ERR_UNSUPPORTED;
    VecRef wv{w, w_dtype == ODIN_BF16};
    if (out_dtype == ODIN_BF16)
        odin_launch(head_unit_scale_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, s, o, wv, w_head_stride, gate,
                    gate_stride, eps, (bf16*)out, T, H, dv);
    else if (out_dtype == ODIN_F32)
        odin_launch(head_unit_scale_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, o, wv, w_head_stride, gate,
                    gate_stride, eps, (float*)out, T, H, dv);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}
