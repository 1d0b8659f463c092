// A routed feed-forward (mixture of experts) without a trip to the host:
//   route_top    softmax over the experts' logits in float, the ``top`` largest scores and their experts per token
//   plan         a counting sort of the (token, choice) pairs by expert, and the list of row tiles of every expert
//   gate/up      act[row] = silu(h[token(row)] Wg[e]^T) * (h[token(row)] Wu[e]^T) over the sorted rows
//   down         y[row] = act[row] Wd[e]^T, float
//   combine      out[token] = sum over its choices of weight * y[row of the pair] (+ a shared expert's output)
// The grids of the two products are sized for the worst case (every expert adds at most one partial tile); blocks
// beyond the tiles that the plan counted return at once.  The order of the rows inside an expert's range depends on
// the order in which threads take their places; a row's result does not, and a token's sum is taken in the order of
// its choices.
#define FE_PDL_CLASS 128
#include <math_constants.h>

#include "common.cuh"

using namespace fe;

constexpr int ROUTE_MAX_EXPERTS = 1024;

// One warp per token.  ties go to the lower expert index.
__global__ void route_top_kernel(const float* __restrict__ logits, int* __restrict__ chosen, float* __restrict__ weights,
                                 int T, int experts, int top, float scale) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float rows[];               // [warps][experts]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + w;
    if (t >= T) return;
    float* s = rows + (size_t)w * experts;
    const float* z = logits + (size_t)t * experts;
    float m = -CUDART_INF_F;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
        const float p = expf(z[e] - m);
        s[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int c = 0; c < top; ++c) {
        float best = -1.f;
        int at = experts;
        for (int e = lane; e < experts; e += 32)
            if (s[e] > best) { best = s[e]; at = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            chosen[(size_t)t * top + c] = at;
            weights[(size_t)t * top + c] = best / sum * scale;
            s[at] = -2.f;
        }
        __syncwarp();
    }
}

extern "C" int fe_route_top(const float* logits, int* chosen, float* weights, int T, int experts, int top, float scale,
                            cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && experts >= 1 && experts <= ROUTE_MAX_EXPERTS && top >= 1 && top <= experts,
               "route_top: bad sizes (experts %d, top %d; at most %d experts)", experts, top, ROUTE_MAX_EXPERTS);
    if (T == 0) return 0;
    const int warps = 4;
    fe::launch(route_top_kernel, (T + warps - 1) / warps, warps * 32, (size_t)warps * experts * sizeof(float), stream, logits,
               chosen, weights, T, experts, top, scale);
    return fe_check_launch("route_top");
}

// One block.  pairs = T * top.  Outputs: offsets[experts + 1] (rows of expert e are offsets[e] .. offsets[e+1]),
// row_of_pair[pairs], pair_of_row[pairs], and the tiles of ``tile_rows`` rows: tile_expert[], tile_row0[], with
// tiles[0] = how many there are.
__global__ void route_plan_kernel(const int* __restrict__ chosen, int pairs, int experts, int tile_rows, int* __restrict__ offsets,
                                  int* __restrict__ row_of_pair, int* __restrict__ pair_of_row, int* __restrict__ tiles,
                                  int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ int count[ROUTE_MAX_EXPERTS];
    __shared__ int cursor[ROUTE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
        else if (status) atomicOr(status, FE_STATUS_BAD_SLOT);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, n = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
                tile_expert[n] = e;
                tile_row0[n] = at + r0;
                ++n;
            }
            at += count[e];
        }
        offsets[experts] = at;
        tiles[0] = n;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= experts) { row_of_pair[p] = -1; continue; }
        const int row = atomicAdd(&cursor[e], 1);
        row_of_pair[p] = row;
        pair_of_row[row] = p;
    }
}

// The two grouped products.  Tile 64 rows x 64 columns, 16 of K a stage, 256 threads with 4 x 4 outputs each; float
// accumulation in ascending k.  GATED: columns n and n + F of the expert's matrix are taken together and
// silu(gate) * up is written (compute type); otherwise the plain product is written in float.
namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
routed_product_kernel(const T* __restrict__ A, const int* __restrict__ pair_of_row, int top, const T* __restrict__ W,
                      void* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tiles,
                      const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int N, int K) {
    griddep_wait();
    griddep_launch_dependents();
    if ((int)blockIdx.y >= tiles[0]) return;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[GATED ? BK : 1][BN + 4];
    __shared__ int source[BM];
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(BM, offsets[e + 1] - row0);
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    // which row of A a sorted row reads: the token of its pair (first product), or the sorted row itself (second)
    if (tid < BM) source[tid] = tid < rows ? (pair_of_row ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const T* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[TM][TN], acu[GATED ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (GATED) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, c = idx % BK;
            const int gk = k0 + c, gn = n0 + r;
            const int src = source[r];
            As[c][r] = (src >= 0 && gk < K) ? to_float(A[(size_t)src * K + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_float(We[(size_t)gn * K + gk]) : 0.f;
            if (GATED) Us[c][r] = (gn < N && gk < K) ? to_float(We[(size_t)(N + gn) * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                w[j] = Ws[k][tx * TN + j];
                if (GATED) u[j] = Us[k][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (GATED) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            const size_t at = (size_t)(row0 + r) * N + gn;
            if (GATED) {
                const float g = acc[i][j];
                reinterpret_cast<T*>(out)[at] = from_float<T>(g / (1.f + expf(-g)) * acu[i][j]);
            } else {
                reinterpret_cast<float*>(out)[at] = acc[i][j];
            }
        }
    }
}

// out[t] = sum_c weights[t][c] * y[row_of_pair[t top + c]] (+ shared[t])
template <typename T>
__global__ void routed_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair,
                                      const float* __restrict__ weights, const T* __restrict__ shared, T* __restrict__ out,
                                      int top, int D) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float total = 0.f;
        for (int c = 0; c < top; ++c) {
            const int row = row_of_pair[(size_t)t * top + c];
            if (row >= 0) total = fmaf(weights[(size_t)t * top + c], y[(size_t)row * D + j], total);
        }
        if (shared) total += to_float(shared[(size_t)t * D + j]);
        out[(size_t)t * D + j] = from_float<T>(total);
    }
}
}  // namespace

extern "C" long long fe_routed_experts_workspace(int T, int top, int experts, int D, int F, int dtype) {
    const long long pairs = (long long)T * top;
    const long long tiles = (pairs + BM - 1) / BM + experts;
    const long long ints = (experts + 1) + 2 * pairs + 1 + 2 * tiles;
    const long long width = dtype == FE_F32 ? 4 : 2;
    return ((ints * 4 + 255) / 256 + (pairs * F * width + 255) / 256 + (pairs * D * 4 + 255) / 256) * 256;
}

// h [T, D]; chosen, weights [T, top]; gate_up [experts, 2F, D]; down [experts, D, F]; shared [T, D] or null; out [T, D].
extern "C" int fe_routed_experts(const void* h, const int* chosen, const float* weights, const void* gate_up, const void* down,
                                 const void* shared, void* out, void* workspace, long long workspace_bytes, int T, int top,
                                 int experts, int D, int F, int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && top >= 1 && experts >= 1 && experts <= ROUTE_MAX_EXPERTS && D > 0 && F > 0, "routed_experts: bad sizes");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "routed_experts: unknown dtype %d", dtype);
    if (T == 0) return 0;
    FE_REQUIRE(workspace_bytes >= fe_routed_experts_workspace(T, top, experts, D, F, dtype), "routed_experts: workspace too small");
    const long long pairs = (long long)T * top;
    const int max_tiles = (int)((pairs + BM - 1) / BM + experts);
    FE_REQUIRE(max_tiles <= 65535, "routed_experts: too many rows in one step (%lld pairs)", pairs);
    int* offsets = (int*)workspace;
    int* row_of_pair = offsets + experts + 1;
    int* pair_of_row = row_of_pair + pairs;
    int* tiles = pair_of_row + pairs;
    int* tile_expert = tiles + 1;
    int* tile_row0 = tile_expert + max_tiles;
    const long long ints = (experts + 1) + 2 * pairs + 1 + 2 * (long long)max_tiles;
    char* act = (char*)workspace + (ints * 4 + 255) / 256 * 256;
    const long long width = dtype == FE_F32 ? 4 : 2;
    float* y = (float*)(act + (pairs * F * width + 255) / 256 * 256);
    fe::launch(route_plan_kernel, 1, 256, 0, stream, chosen, (int)pairs, experts, BM, offsets, row_of_pair, pair_of_row, tiles,
               tile_expert, tile_row0, status);
    const dim3 grid1((F + BN - 1) / BN, max_tiles), grid2((D + BN - 1) / BN, max_tiles);
    const int threads = D >= 1024 ? 256 : 128;
    if (dtype == FE_F32) {
        fe::launch(routed_product_kernel<float, true>, grid1, 256, 0, stream, (const float*)h, (const int*)pair_of_row, top,
                   (const float*)gate_up, (void*)act, (const int*)offsets, (const int*)tiles, (const int*)tile_expert,
                   (const int*)tile_row0, F, D);
        fe::launch(routed_product_kernel<float, false>, grid2, 256, 0, stream, (const float*)act, (const int*)nullptr, top,
                   (const float*)down, (void*)y, (const int*)offsets, (const int*)tiles, (const int*)tile_expert,
                   (const int*)tile_row0, D, F);
        fe::launch(routed_combine_kernel<float>, T, threads, 0, stream, (const float*)y, (const int*)row_of_pair, weights,
                   (const float*)shared, (float*)out, top, D);
    } else {
        fe::launch(routed_product_kernel<bf16, true>, grid1, 256, 0, stream, (const bf16*)h, (const int*)pair_of_row, top,
                   (const bf16*)gate_up, (void*)act, (const int*)offsets, (const int*)tiles, (const int*)tile_expert,
                   (const int*)tile_row0, F, D);
        fe::launch(routed_product_kernel<bf16, false>, grid2, 256, 0, stream, (const bf16*)act, (const int*)nullptr, top,
                   (const bf16*)down, (void*)y, (const int*)offsets, (const int*)tiles, (const int*)tile_expert,
                   (const int*)tile_row0, D, F);
        fe::launch(routed_combine_kernel<bf16>, T, threads, 0, stream, (const float*)y, (const int*)row_of_pair, weights,
                   (const bf16*)shared, (bf16*)out, top, D);
    }
    return fe_check_launch("routed_experts");
}
