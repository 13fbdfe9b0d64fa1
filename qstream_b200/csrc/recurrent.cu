// Mixers that carry a matrix of state per head from token to token, and the token shift in front of one of them.
//
//   linear attention with a fixed decay per head ("lightning"):
//       S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t                   q, k [dk], v, o [dv], S [dk, dv]
//   time mixing with a decay per token and key channel and a bonus for the current token ("wkv"):
//       o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T,   w_t = exp(-exp(d_t))
//
// The state lives in 32-bit, per slot as [heads][dv][dk] (a column of S is contiguous), starts at zero and is
// read at the start of a step and written back at its end; everything between the projections and the output is
// 32-bit arithmetic.  One kernel serves prompts and single tokens: a block owns some columns of one head of one
// sequence and walks the sequence's tokens of this step in order.  A thread owns RK consecutive key rows of one
// column; the KS threads of a column are neighbours in a warp and add their parts of o by shuffles, in a fixed
// order, so a token's result does not depend on the batch or on how the prompt was cut.
#include "common.cuh"

namespace {

constexpr int RK = 32;              // key rows per thread
constexpr int TILE = 8;             // tokens staged in shared memory at a time

template <typename TI, bool WKV>
__global__ void __launch_bounds__(256)
state_scan_kernel(float* __restrict__ o, size_t ldo,
                  const TI* __restrict__ q, size_t ldq, const TI* __restrict__ k, size_t ldk,
                  const TI* __restrict__ v, size_t ldv, const float* __restrict__ dlog, size_t ldd,
                  const float* __restrict__ head_decay, const void* __restrict__ bonus, int bonus_dtype,
                  float* __restrict__ state, size_t slot_stride,
                  const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot, int n_seq, int T_rows,
                  int H, int dk, int dv, int ks_log2, int cols, int in_act) {
    extern __shared__ float smem[];
    const int KS = 1 << ks_log2, dkp = KS * RK;
    float* sq = smem;                                   // [TILE][dkp]
    float* sk = sq + TILE * dkp;                        // [TILE][dkp]
    float* sw = sk + TILE * dkp;                        // [TILE][dkp]   (WKV only)
    float* sv = sw + (WKV ? TILE * dkp : 0);            // [TILE][cols]
    grid_dep_launch();
    grid_dep_wait();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols;
    const int n_cols = min(cols, dv - col0);
    const int tid = threadIdx.x;
    // rows of the packed batch beyond the last sequence belong to nobody: give them a defined value
    if (s == 0) {
        for (int t = seq_start[n_seq]; t < T_rows; ++t)
            for (int c = tid; c < n_cols; c += blockDim.x) o[(size_t)t * ldo + h * dv + col0 + c] = 0.f;
    }
    const int slot = seq_slot[s];
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (slot < 0) {
        for (int t = t0; t < t1; ++t)
            for (int c = tid; c < n_cols; c += blockDim.x) o[(size_t)t * ldo + h * dv + col0 + c] = 0.f;
        return;
    }
    if (t1 <= t0) return;
    const int col = tid >> ks_log2, ks = tid & (KS - 1);
    const bool owner = col < n_cols;
    const int i0 = ks * RK;
    float* scol = state + (size_t)slot * slot_stride + ((size_t)h * dv + col0 + (owner ? col : 0)) * dk;

    float S[RK], u[RK];
#pragma unroll
    for (int r = 0; r < RK; ++r) {
        S[r] = (owner && i0 + r < dk) ? scol[i0 + r] : 0.f;
        u[r] = (WKV && i0 + r < dk) ? load_as_f32(bonus, bonus_dtype, (size_t)h * dk + i0 + r) : 0.f;
    }
    const float decay = WKV ? 0.f : head_decay[h];

    for (int base = t0; base < t1; base += TILE) {
        const int nt = min(TILE, t1 - base);
        __syncthreads();
        for (int e = tid; e < nt * dkp; e += blockDim.x) {
            const int tt = e / dkp, i = e - tt * dkp;
            const size_t row = (size_t)(base + tt);
            float qv = 0.f, kv = 0.f, wv = 0.f;
            if (i < dk) {
                qv = apply_activation(to_f32(q[row * ldq + h * dk + i]), in_act);
                kv = apply_activation(to_f32(k[row * ldk + h * dk + i]), in_act);
                if (WKV) wv = expf(-expf(dlog[row * ldd + h * dk + i]));
            }
            sq[e] = qv;
            sk[e] = kv;
            if (WKV) sw[e] = wv;
        }
        for (int e = tid; e < nt * cols; e += blockDim.x) {
            const int tt = e / cols, c = e - tt * cols;
            sv[e] = c < n_cols ? apply_activation(to_f32(v[(size_t)(base + tt) * ldv + h * dv + col0 + c]), in_act) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = sv[tt * cols + (owner ? col : 0)];
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * dkp + i0);
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * dkp + i0);
            const float4* w4 = reinterpret_cast<const float4*>(sw + tt * dkp + i0);
            float acc = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < RK / 4; ++r4) {
                const float4 qq = q4[r4], kk = k4[r4];
                const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w};
                float wa[4] = {0.f, 0.f, 0.f, 0.f};
                if (WKV) { const float4 ww = w4[r4]; wa[0] = ww.x; wa[1] = ww.y; wa[2] = ww.z; wa[3] = ww.w; }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    const float kv = ka[j] * vj;
                    if (WKV) {
                        acc = fmaf(qa[j], fmaf(u[r], kv, S[r]), acc);
                        S[r] = fmaf(wa[j], S[r], kv);
                    } else {
                        S[r] = fmaf(decay, S[r], kv);
                        acc = fmaf(qa[j], S[r], acc);
                    }
                }
            }
            for (int off = KS >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (owner && ks == 0) o[(size_t)(base + tt) * ldo + h * dv + col0 + col] = acc;
        }
    }
    if (owner) {
#pragma unroll
        for (int r = 0; r < RK; ++r)
            if (i0 + r < dk) scol[i0 + r] = S[r];
    }
}

// ----------------------------------------------------------------------------- token shift

// out[m][t] = h[t] + (h[t-1] - h[t]) * mu[m], m < n_mix; h[t-1] is zero for a sequence's first token, the row
// above inside a step, and what the earlier steps left in `last_row[slot]` for the first row of a later step.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, size_t ldo, size_t mix_stride, const T* __restrict__ h, size_t ldh,
                                   const float* __restrict__ mu, const T* __restrict__ last_row, size_t ld_last,
                                   const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                   int D, int n_mix) {
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    const T* before = nullptr;
    if (slot >= 0 && tok_pos[t] > 0)
        before = (t > 0 && tok_slot[t - 1] == slot) ? h + (size_t)(t - 1) * ldh : last_row + (size_t)slot * ld_last;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float cur = slot >= 0 ? to_f32(h[(size_t)t * ldh + i]) : 0.f;
        const float diff = (before ? to_f32(before[i]) : 0.f) - cur;
        for (int m = 0; m < n_mix; ++m)
            out[(size_t)m * mix_stride + (size_t)t * ldo + i] = from_f32<T>(fmaf(diff, mu[(size_t)m * D + i], cur));
    }
}

template <typename TI>
int launch_scan(bool wkv, float* o, long long ldo, const void* q, long long ldq, const void* k, long long ldk, const void* v,
                long long ldv, const float* dlog, long long ldd, const float* head_decay, const void* bonus, int bonus_dtype,
                float* state, long long slot_stride, const int32_t* seq_start, const int32_t* seq_slot, int n_seq, int T_rows,
                int H, int dk, int dv, int in_act, cudaStream_t stream) {
    int ks_log2 = 0;
    while ((RK << ks_log2) < dk) ++ks_log2;
    const int KS = 1 << ks_log2;
    int cols = 256 / KS;
    if (cols > dv) cols = dv;
    // few sequences and heads: narrower blocks, so that more SMs take part
    while (cols > 8 && (long long)n_seq * H * ((dv + cols - 1) / cols) < 148 && cols * KS > 64) cols >>= 1;
    const int threads = ((cols * KS + 31) / 32) * 32;
    const int dkp = KS * RK;
    const size_t smem = (size_t)TILE * ((wkv ? 3 : 2) * dkp + cols) * sizeof(float);
    dim3 grid(n_seq, H, (dv + cols - 1) / cols);
    cudaError_t e;
    if (wkv)
        e = qs_launch_dependent(state_scan_kernel<TI, true>, grid, dim3(threads), smem, stream, o, (size_t)ldo, (const TI*)q,
                                (size_t)ldq, (const TI*)k, (size_t)ldk, (const TI*)v, (size_t)ldv, dlog, (size_t)ldd, head_decay,
                                bonus, bonus_dtype, state, (size_t)slot_stride, seq_start, seq_slot, n_seq, T_rows, H, dk, dv,
                                ks_log2, cols, in_act);
    else
        e = qs_launch_dependent(state_scan_kernel<TI, false>, grid, dim3(threads), smem, stream, o, (size_t)ldo, (const TI*)q,
                                (size_t)ldq, (const TI*)k, (size_t)ldk, (const TI*)v, (size_t)ldv, dlog, (size_t)ldd, head_decay,
                                bonus, bonus_dtype, state, (size_t)slot_stride, seq_start, seq_slot, n_seq, T_rows, H, dk, dv,
                                ks_log2, cols, in_act);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "state_scan: %s", cudaGetErrorString(e));
    return qs_check_launch("state_scan");
}

}  // namespace

// mode 0: fixed decay per head (`head_decay` [H], float32 on the device); mode 1: decay exp(-exp(dlog)) per token and
// key channel (`dlog` [T, H * dk] float32) and the bonus `bonus` [H, dk] for the current token.
// q, k [T, H * dk] and v [T, H * dv] of type `dtype`, with `in_act` applied on the way in; o [T, H * dv] float32;
// state [slots][H][dv][dk] float32 with `slot_stride` floats between slots.
QS_API int qs_state_scan(int mode, float* o, long long ldo, const void* q, long long ldq, const void* k, long long ldk,
                         const void* v, long long ldv, int dtype, const float* dlog, long long ldd, const float* head_decay,
                         const void* bonus, int bonus_dtype, float* state, long long slot_stride, const int32_t* seq_start,
                         const int32_t* seq_slot, int n_seq, int T_rows, int H, int dk, int dv, int in_act,
                         cudaStream_t stream) {
    if (n_seq == 0 || T_rows == 0) return QS_OK;
    QS_REQUIRE(n_seq > 0 && T_rows > 0 && H > 0 && dk > 0 && dv > 0, "state_scan: bad sizes");
    QS_REQUIRE(dk <= 8 * RK, "state_scan: %d key channels per head above %d", dk, 8 * RK);
    QS_REQUIRE(H <= 65535, "state_scan: %d heads exceed the grid", H);
    QS_REQUIRE(mode == 0 ? head_decay != nullptr : (mode == 1 && dlog && bonus), "state_scan: mode %d lacks its operands", mode);
    if (dtype == QS_F32)
        return launch_scan<float>(mode == 1, o, ldo, q, ldq, k, ldk, v, ldv, dlog, ldd, head_decay, bonus, bonus_dtype, state,
                                  slot_stride, seq_start, seq_slot, n_seq, T_rows, H, dk, dv, in_act, stream);
    if (dtype == QS_BF16)
        return launch_scan<__nv_bfloat16>(mode == 1, o, ldo, q, ldq, k, ldk, v, ldv, dlog, ldd, head_decay, bonus, bonus_dtype,
                                          state, slot_stride, seq_start, seq_slot, n_seq, T_rows, H, dk, dv, in_act, stream);
    return qs_fail(QS_ERR_INVALID_INPUT, "state_scan: unknown dtype %d", dtype);
}

QS_API int qs_token_shift(void* out, long long ldo, long long mix_stride, const void* h, long long ldh, int dtype,
                          const float* mu, const void* last_row, long long ld_last, const int32_t* tok_slot,
                          const int32_t* tok_pos, int T, int D, int n_mix, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && D > 0 && n_mix > 0, "token_shift: bad sizes");
    const int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == QS_F32)
        e = qs_launch_dependent(token_shift_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)out, (size_t)ldo,
                                (size_t)mix_stride, (const float*)h, (size_t)ldh, mu, (const float*)last_row, (size_t)ld_last,
                                tok_slot, tok_pos, D, n_mix);
    else if (dtype == QS_BF16)
        e = qs_launch_dependent(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)out,
                                (size_t)ldo, (size_t)mix_stride, (const __nv_bfloat16*)h, (size_t)ldh, mu,
                                (const __nv_bfloat16*)last_row, (size_t)ld_last, tok_slot, tok_pos, D, n_mix);
    else return qs_fail(QS_ERR_INVALID_INPUT, "token_shift: unknown dtype %d", dtype);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "token_shift: %s", cudaGetErrorString(e));
    return qs_check_launch("token_shift");
}
