// A linear-recurrent mixer with a matrix state per head (key channel x value channel) and a decay per key channel
// that depends on the token:
//   blends   x_s = h + (h' - h) * mu_s, h' the row of the token before (s = r, k, v, g, w)
//   decay    w_t = exp(-exp(logit_t + w0))                              (float)
//   output   o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])
//   state    S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]                  (float, carried from step to step per request)
//   finish   y = o / rms(o per head) * weight * silu(g)
// The projections r, k, v, g come in the compute type; everything else here is float.
#define FE_PDL_CLASS 128
#include "common.cuh"

using namespace fe;

// ---------------------------------------------------------------------------------------------
// One block per token.  ``state`` rows are seats; the kept row of a seat (the last normalised input of the step before)
// starts at ``offset`` floats into its row.  The block of a request's first token reads the kept row and writes the
// request's last row of this step in its place, element by element in the same thread, so nobody else touches it.
template <typename T>
__global__ void token_shift_blend_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* state,
                                         long long state_stride, long long offset, const int* __restrict__ seats,
                                         const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                         T* __restrict__ blends, float* __restrict__ blend_w, int T_tokens, int D, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    const int r = token_req[t];
    const int first = cu_q[r];
    const int seat = seats[r];
    const bool seated = seat >= 0 && seat < n_seats;
    float* kept = seated ? state + (size_t)seat * state_stride + offset : nullptr;
    const T* row = h + (size_t)t * D;
    const T* prev = t > first ? h + (size_t)(t - 1) * D : nullptr;
    const T* last = h + (size_t)(cu_q[r + 1] - 1) * D;
    const size_t plane = (size_t)T_tokens * D;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        const float x = to_float(row[j]);
        float before;
        if (prev) before = to_float(prev[j]);
        else if (kept) {
            before = kept[j];
            kept[j] = to_float(last[j]);
        } else before = 0.f;
        const float diff = before - x;
        const size_t at = (size_t)t * D + j;
#pragma unroll
        for (int s = 0; s < 4; ++s) blends[s * plane + at] = from_float<T>(fmaf(diff, mu[(size_t)s * D + j], x));
        blend_w[at] = fmaf(diff, mu[(size_t)4 * D + j], x);
    }
}

extern "C" int fe_token_shift_blend(const void* h, const float* mu, float* state, long long state_stride, long long offset,
                                    const int* seats, const int* cu_q, const int* token_req, void* blends, float* blend_w,
                                    int T, int D, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && D > 0 && n_seats >= 0 && offset >= 0 && offset + D <= state_stride, "token_shift_blend: bad sizes");
    if (T == 0) return 0;
    const int threads = D >= 1024 ? 256 : 128;
    if (dtype == FE_F32)
        fe::launch(token_shift_blend_kernel<float>, T, threads, 0, stream, (const float*)h, mu, state, state_stride, offset, seats,
                   cu_q, token_req, (float*)blends, blend_w, T, D, n_seats);
    else if (dtype == FE_BF16)
        fe::launch(token_shift_blend_kernel<bf16>, T, threads, 0, stream, (const bf16*)h, mu, state, state_stride, offset, seats,
                   cu_q, token_req, (bf16*)blends, blend_w, T, D, n_seats);
    else
        FE_REQUIRE(false, "token_shift_blend: unknown dtype %d", dtype);
    return fe_check_launch("token_shift_blend");
}

// ---------------------------------------------------------------------------------------------
// The recurrence.  One block per (request, head); thread j owns value channel j and the state column S[.][j]: in
// registers when the head size is one the kernel is compiled for (DH > 0), else in shared memory.  Tokens are walked
// in tiles of TILE: the block stages r, k, the decay and v of a tile in shared memory, then every thread walks the
// tile's tokens over all key channels.  A seat below 0 (a padding request) starts from zero and keeps nothing.
constexpr int WKV_TILE = 16;

template <typename T, int DH>
__global__ void wkv_recurrence_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                      const float* __restrict__ logits, const float* __restrict__ w0,
                                      const float* __restrict__ u, float* state, long long state_stride,
                                      const int* __restrict__ seats, const int* __restrict__ cu_q, float* __restrict__ out,
                                      int heads, int d_runtime, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int d = DH > 0 ? DH : d_runtime;
    extern __shared__ float smem[];
    float* rs = smem;                         // [TILE][d]
    float* ks = rs + WKV_TILE * d;
    float* ws = ks + WKV_TILE * d;
    float* vs = ws + WKV_TILE * d;
    float* us = vs + WKV_TILE * d;            // [d]
    float* bs = us + d;                       // [d]  w0 of this head
    float* column = bs + d;                   // [d][d] when DH == 0
    const int req = blockIdx.x, head = blockIdx.y;
    const int j = threadIdx.x;
    const bool owner = j < d;
    const int seat = seats[req];
    const bool seated = seat >= 0 && seat < n_seats;
    float* mine = seated ? state + (size_t)seat * state_stride + (size_t)head * d * d : nullptr;
    const int inner = heads * d;
    float S[DH > 0 ? DH : 1];
    if (owner) {
        if (DH > 0) {
#pragma unroll
            for (int i = 0; i < (DH > 0 ? DH : 1); ++i) S[i] = mine ? mine[(size_t)i * d + j] : 0.f;
        } else {
            for (int i = 0; i < d; ++i) column[i * d + j] = mine ? mine[(size_t)i * d + j] : 0.f;
        }
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        us[i] = u[head * d + i];
        bs[i] = w0[head * d + i];
    }
    __syncthreads();
    const int begin = cu_q[req], end = cu_q[req + 1];
    for (int t0 = begin; t0 < end; t0 += WKV_TILE) {
        const int count = min(WKV_TILE, end - t0);
        for (int e = threadIdx.x; e < count * d; e += blockDim.x) {
            const int tt = e / d, i = e % d;
            const size_t at = (size_t)(t0 + tt) * inner + (size_t)head * d + i;
            rs[e] = to_float(r[at]);
            ks[e] = to_float(k[at]);
            vs[e] = to_float(v[at]);
            ws[e] = expf(-expf(logits[at] + bs[i]));
        }
        __syncthreads();
        if (owner) {
            for (int tt = 0; tt < count; ++tt) {
                const float vj = vs[tt * d + j];
                const float* rt = rs + tt * d;
                const float* kt = ks + tt * d;
                const float* wt = ws + tt * d;
                float acc = 0.f;
                if (DH > 0) {
#pragma unroll
                    for (int i = 0; i < (DH > 0 ? DH : 1); ++i) {
                        const float kv = kt[i] * vj;
                        acc = fmaf(rt[i], fmaf(us[i], kv, S[i]), acc);
                        S[i] = fmaf(wt[i], S[i], kv);
                    }
                } else {
                    for (int i = 0; i < d; ++i) {
                        const float kv = kt[i] * vj;
                        const float s = column[i * d + j];
                        acc = fmaf(rt[i], fmaf(us[i], kv, s), acc);
                        column[i * d + j] = fmaf(wt[i], s, kv);
                    }
                }
                out[(size_t)(t0 + tt) * inner + (size_t)head * d + j] = acc;
            }
        }
        __syncthreads();
    }
    if (owner && mine) {
        if (DH > 0) {
#pragma unroll
            for (int i = 0; i < (DH > 0 ? DH : 1); ++i) mine[(size_t)i * d + j] = S[i];
        } else {
            for (int i = 0; i < d; ++i) mine[(size_t)i * d + j] = column[i * d + j];
        }
    }
}

template <typename T, int DH>
static int launch_wkv(const void* r, const void* k, const void* v, const float* logits, const float* w0, const float* u,
                      float* state, long long state_stride, const int* seats, const int* cu_q, float* out, int requests,
                      int heads, int d, int n_seats, cudaStream_t stream) {
    const int threads = (d + 31) / 32 * 32;
    size_t smem = ((size_t)4 * WKV_TILE * d + 2 * d) * sizeof(float);
    if (DH == 0) smem += (size_t)d * d * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(wkv_recurrence_kernel<T, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "wkv_recurrence: %s", cudaGetErrorString(err));
    }
    fe::launch(wkv_recurrence_kernel<T, DH>, dim3(requests, heads), threads, smem, stream, (const T*)r, (const T*)k, (const T*)v,
               logits, w0, u, state, state_stride, seats, cu_q, out, heads, d, n_seats);
    return fe_check_launch("wkv_recurrence");
}

template <typename T>
static int dispatch_wkv(const void* r, const void* k, const void* v, const float* logits, const float* w0, const float* u,
                        float* state, long long state_stride, const int* seats, const int* cu_q, float* out, int requests,
                        int heads, int d, int n_seats, cudaStream_t stream) {
#define FE_WKV(DH) return launch_wkv<T, DH>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream)
    switch (d) {
        case 32: FE_WKV(32);
        case 64: FE_WKV(64);
        case 128: FE_WKV(128);
        default: FE_WKV(0);
    }
#undef FE_WKV
}

extern "C" int fe_wkv_recurrence(const void* r, const void* k, const void* v, const float* logits, const float* w0,
                                 const float* u, float* state, long long state_stride, const int* seats, const int* cu_q,
                                 float* out, int requests, int heads, int d, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && heads > 0 && d > 0 && d <= 192 && n_seats >= 0 && (long long)heads * d * d <= state_stride,
               "wkv_recurrence: bad sizes (heads %d, head size %d; head sizes up to 192)", heads, d);
    FE_REQUIRE(heads <= 65535, "wkv_recurrence: too many heads (%d)", heads);
    if (requests == 0) return 0;
    if (dtype == FE_F32)
        return dispatch_wkv<float>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream);
    if (dtype == FE_BF16)
        return dispatch_wkv<bf16>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream);
    FE_REQUIRE(false, "wkv_recurrence: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// y[t, head] = o[t, head] / sqrt(mean(o[t, head]^2) + eps) * weight * silu(g): one warp per (token, head).
template <typename T>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, const T* __restrict__ g,
                                         T* __restrict__ out, float eps, long long pairs, int heads, int d) {
    griddep_wait();
    griddep_launch_dependents();
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (warp >= pairs) return;
    const int lane = threadIdx.x & 31;
    const int head = (int)(warp % heads);
    const float* x = o + warp * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) {
        const float gate = to_float(g[warp * d + i]);
        out[warp * d + i] = from_float<T>(x[i] * inv * weight[head * d + i] * (gate / (1.f + expf(-gate))));
    }
}

extern "C" int fe_head_rmsnorm_gate(const float* o, const float* weight, const void* g, void* out, float eps, int T, int heads,
                                    int d, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && d > 0, "head_rmsnorm_gate: bad sizes");
    if (T == 0) return 0;
    const long long pairs = (long long)T * heads;
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    if (dtype == FE_F32)
        fe::launch(head_rmsnorm_gate_kernel<float>, blocks, 128, 0, stream, o, weight, (const float*)g, (float*)out, eps, pairs, heads, d);
    else if (dtype == FE_BF16)
        fe::launch(head_rmsnorm_gate_kernel<bf16>, blocks, 128, 0, stream, o, weight, (const bf16*)g, (bf16*)out, eps, pairs, heads, d);
    else
        FE_REQUIRE(false, "head_rmsnorm_gate: unknown dtype %d", dtype);
    return fe_check_launch("head_rmsnorm_gate");
}
