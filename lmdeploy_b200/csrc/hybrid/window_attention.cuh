// Kernels of pre-norm hybrid blocks: table rows added to the stream, residual add fused with an RMS norm, softmax attention
// with grouped key/value heads over a sliding window of a paged cache (capped scores, a logarithmic distance penalty, the
// heads' weight rows recombined by a matrix after the softmax, an output gate), and the squared-relu activation.
// Included by hybrid_ops.cu inside namespace b200h, after its helpers (to_f / from_f / block_sum / sigmoid_f).
//
// Cache entry of position p of a sequence, inside its page (page address + layer_off): the normed key as T at
// [p % block_len][kv_heads * dim], and, v_off bytes further, the value as T at [p % block_len][kv_heads * vdim].
//
// Attention runs in two passes over a row's visible keys [max(0, pos - window + 1), pos], both cut into `splits` equal key
// ranges so that a step of few rows still fills the SMs:
//   pass 1 (window_stats_kernel, one block per row, key/value head and range): scores of the heads that share the key/value
//          head, their running maximum and denominator;
//   pass 2 (window_pv_kernel, one block per row and range): the ranges' (maximum, denominator) pairs are merged per head, the
//          scores are computed again for ALL heads of the row, turned into final softmax weights, recombined across heads
//          (weight'_h = sum_g talk[h, g] weight_g -- this couples every head of a row, hence one block for all of them) and
//          applied to the values of each head's own key/value head;
//   window_out_kernel sums the ranges' partial outputs, applies sigmoid(gate) and writes T.
// Scores, softmax, recombination and the weighted value sums are float whatever T is.

constexpr int kMaxRep = 8;              // query heads of one key/value head handled per walk over a key
constexpr int kWinTile = 32;            // keys per tile of pass 2

// x[t] += table[idx ? idx[t] : fixed]
template <typename T>
__global__ void add_rows_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ idx, int fixed, int width)
{
    const int t = blockIdx.x;
    const T* row = table + (size_t)(idx ? idx[t] : fixed) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] += to_f(row[i]);
}

// x[t] += m[t] (+ extra); h[t] = x[t] / rms(x[t]) * w.  m, extra and h are optional.
template <typename T>
__global__ void residual_norm_kernel(float* __restrict__ x, const T* __restrict__ m, const T* __restrict__ extra,
                                     const float* __restrict__ w, int width, float eps, float* __restrict__ h)
{
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = x[base + i];
        if (m) v += to_f(m[base + i]);
        if (extra) v += to_f(extra[i]);
        if (m || extra) x[base + i] = v;
        ss += v * v;
    }
    if (!h) return;
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) h[base + i] = x[base + i] * r * w[i];
}

// x <- relu(x)^2 in place
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = fmaxf(to_f(x[i]), 0.f);
    x[i] = from_f<T>(v * v);
}

// One block per row: the query is normed over all its heads at once (-> qn, float), the key likewise and written to the row's
// cache entry as T, the value is copied to the cache.  wq / wk == nullptr: no norm of that projection.
template <typename T>
__global__ void window_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int64_t ld, int q_cols,
                                   int k_cols, int v_cols, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int64_t* __restrict__ block_ptrs,
                                   const int* __restrict__ cu_blocks, int64_t layer_off, int64_t v_off, int block_len,
                                   float* __restrict__ qn)
{
    __shared__ float red[32];
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t];
    const T* qr = q + (size_t)t * ld;
    float r = 1.0f;
    if (wq) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_cols; i += blockDim.x) { const float a = to_f(qr[i]); ss += a * a; }
        ss = block_sum(ss, red);
        r = 1.0f / sqrtf(ss / (float)q_cols + eps);
    }
    for (int i = threadIdx.x; i < q_cols; i += blockDim.x) qn[(size_t)t * q_cols + i] = wq ? to_f(qr[i]) * r * wq[i] : to_f(qr[i]);

    char* page = reinterpret_cast<char*>(block_ptrs[cu_blocks[s] + pos / block_len]) + layer_off;
    const int at = pos % block_len;
    const T* kr = k + (size_t)t * ld;
    T* k_dst = reinterpret_cast<T*>(page) + (size_t)at * k_cols;
    r = 1.0f;
    if (wk) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < k_cols; i += blockDim.x) { const float a = to_f(kr[i]); ss += a * a; }
        ss = block_sum(ss, red);
        r = 1.0f / sqrtf(ss / (float)k_cols + eps);
    }
    for (int i = threadIdx.x; i < k_cols; i += blockDim.x) k_dst[i] = wk ? from_f<T>(to_f(kr[i]) * r * wk[i]) : kr[i];
    const T* vr = v + (size_t)t * ld;
    T* v_dst = reinterpret_cast<T*>(page + v_off) + (size_t)at * v_cols;
    for (int i = threadIdx.x; i < v_cols; i += blockDim.x) v_dst[i] = vr[i];
}

struct WindowGeom {
    int heads, kv_heads, dim, vdim, block_len, window, splits;
    float scale, softcap;
    const float* r1;          // [heads] or nullptr: no distance penalty
    const float* r2;
    const float* talk;        // [heads, heads] or nullptr: heads are not recombined
    const int* tok_seq;
    const int* tok_pos;
    const int64_t* block_ptrs;
    const int* cu_blocks;
    int64_t layer_off, v_off;
};

// The key range `z` of a row at position pos: [j0, j1).
__device__ __forceinline__ void window_range(const WindowGeom& g, int pos, int z, int& j0, int& j1)
{
    const int lo = g.window > 0 ? max(0, pos - g.window + 1) : 0;
    const int per = (pos - lo + g.splits) / g.splits;         // ceil((pos - lo + 1) / splits)
    j0 = lo + z * per;
    j1 = min(pos + 1, j0 + per);
}

// score of head `head` for a key at distance `dist` behind the query, from the raw dot product
__device__ __forceinline__ float window_score(const WindowGeom& g, float dot, int head, int dist)
{
    float s = dot * g.scale;
    if (g.softcap > 0.f) s = g.softcap * tanhf(s / g.softcap);
    if (g.r1) s -= g.r1[head] * log1pf(g.r2[head] * (float)dist);
    return s;
}

// dot products of one cached key with `cnt` (<= kMaxRep) queries that lie `dim` floats apart in shared memory
template <typename T, bool VEC>
__device__ __forceinline__ void key_dots(const T* __restrict__ key, const float* __restrict__ qs, int dim, int cnt, float* acc)
{
#pragma unroll
    for (int u = 0; u < kMaxRep; ++u) acc[u] = 0.f;
    if (VEC) {
        constexpr int N = 16 / (int)sizeof(T);
        for (int d = 0; d < dim; d += N) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + d);
            const T* e = reinterpret_cast<const T*>(&raw);
            float kv[N];
#pragma unroll
            for (int i = 0; i < N; ++i) kv[i] = to_f(e[i]);
#pragma unroll
            for (int u = 0; u < kMaxRep; ++u) {
                if (u < cnt) {
                    const float* qu = qs + u * dim + d;
#pragma unroll
                    for (int i = 0; i < N; ++i) acc[u] = fmaf(qu[i], kv[i], acc[u]);
                }
            }
        }
    } else {
        for (int d = 0; d < dim; ++d) {
            const float kv = to_f(key[d]);
#pragma unroll
            for (int u = 0; u < kMaxRep; ++u)
                if (u < cnt) acc[u] = fmaf(qs[u * dim + d], kv, acc[u]);
        }
    }
}

__device__ __forceinline__ const char* window_page(const WindowGeom& g, const int64_t* pages, int j)
{
    return reinterpret_cast<const char*>(pages[j / g.block_len]) + g.layer_off;
}

// (m, l) <- merge of two running (maximum, denominator) pairs
__device__ __forceinline__ void merge_ml(float& m, float& l, float om, float ol)
{
    const float mx = fmaxf(m, om);
    l = l * expf(m - mx) + ol * expf(om - mx);
    m = mx;
}

// Pass 1.  grid (rows, kv_heads, splits), 128 threads: thread i walks keys j0 + i, j0 + i + 128, ... of the range.
template <typename T, bool VEC>
__global__ void __launch_bounds__(128) window_stats_kernel(const float* __restrict__ qn, WindowGeom g, float* __restrict__ ml)
{
    extern __shared__ __align__(16) float win_smem[];
    __shared__ float red_m[4][kMaxRep], red_l[4][kMaxRep];
    const int t = blockIdx.x, c = blockIdx.y, z = blockIdx.z, tid = threadIdx.x;
    const int rep = g.heads / g.kv_heads, s = g.tok_seq[t], pos = g.tok_pos[t];
    float* qs = win_smem;                                                    // [rep][dim]
    const float* qrow = qn + ((size_t)t * g.heads + (size_t)c * rep) * g.dim;
    for (int i = tid; i < rep * g.dim; i += blockDim.x) qs[i] = qrow[i];
    __syncthreads();
    int j0, j1;
    window_range(g, pos, z, j0, j1);
    const int64_t* pages = g.block_ptrs + g.cu_blocks[s];
    const size_t k_row = (size_t)g.kv_heads * g.dim;
    for (int hb = 0; hb < rep; hb += kMaxRep) {
        const int cnt = min(kMaxRep, rep - hb);
        float m[kMaxRep], l[kMaxRep];
#pragma unroll
        for (int u = 0; u < kMaxRep; ++u) { m[u] = -1e30f; l[u] = 0.f; }
        for (int j = j0 + tid; j < j1; j += blockDim.x) {
            const T* key = reinterpret_cast<const T*>(window_page(g, pages, j)) + (size_t)(j % g.block_len) * k_row + (size_t)c * g.dim;
            float acc[kMaxRep];
            key_dots<T, VEC>(key, qs + hb * g.dim, g.dim, cnt, acc);
#pragma unroll
            for (int u = 0; u < kMaxRep; ++u) {
                if (u < cnt) merge_ml(m[u], l[u], window_score(g, acc[u], c * rep + hb + u, pos - j), 1.0f);
            }
        }
        // across the block: lanes of a warp by shuffles, the four warps through shared memory
#pragma unroll
        for (int u = 0; u < kMaxRep; ++u) {
            for (int o = 16; o > 0; o >>= 1) {
                const float om = __shfl_xor_sync(0xffffffffu, m[u], o), ol = __shfl_xor_sync(0xffffffffu, l[u], o);
                merge_ml(m[u], l[u], om, ol);
            }
        }
        __syncthreads();
        if ((tid & 31) == 0) {
#pragma unroll
            for (int u = 0; u < kMaxRep; ++u) { red_m[tid >> 5][u] = m[u]; red_l[tid >> 5][u] = l[u]; }
        }
        __syncthreads();
        if (tid < cnt) {
            float mm = red_m[0][tid], ll = red_l[0][tid];
            for (int w = 1; w < 4; ++w) merge_ml(mm, ll, red_m[w][tid], red_l[w][tid]);
            float* dst = ml + (((size_t)t * g.heads + c * rep + hb + tid) * g.splits + z) * 2;
            dst[0] = mm;
            dst[1] = ll;
        }
    }
}

// Pass 2.  grid (rows, splits), 256 threads.  Shared memory (floats): qs [heads][dim] | mx [heads] | linv [heads] |
// talk [heads][heads] | p [heads][kWinTile] | p2 [heads][kWinTile] | o [heads][vdim].
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) window_pv_kernel(const float* __restrict__ qn, WindowGeom g, const float* __restrict__ ml,
                                                        float* __restrict__ o_part)
{
    extern __shared__ __align__(16) float win_smem[];
    const int t = blockIdx.x, z = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    const int H = g.heads, G = g.kv_heads, rep = H / G, D = g.dim, V = g.vdim;
    const int s = g.tok_seq[t], pos = g.tok_pos[t];
    float* qs = win_smem;
    float* mx = qs + (size_t)H * D;
    float* linv = mx + H;
    float* talk = linv + H;
    float* p = talk + (g.talk ? H * H : 0);
    float* p2 = g.talk ? p + H * kWinTile : p;
    float* o = p2 + H * kWinTile;
    for (int i = tid; i < H * D; i += nt) qs[i] = qn[(size_t)t * H * D + i];
    for (int i = tid; i < H * V; i += nt) o[i] = 0.f;
    if (g.talk)
        for (int i = tid; i < H * H; i += nt) talk[i] = g.talk[i];
    for (int h = tid; h < H; h += nt) {
        const float* src = ml + ((size_t)t * H + h) * g.splits * 2;
        float mm = src[0], ll = src[1];
        for (int k = 1; k < g.splits; ++k) merge_ml(mm, ll, src[2 * k], src[2 * k + 1]);
        mx[h] = mm;
        linv[h] = 1.0f / ll;
    }
    __syncthreads();
    int j0, j1;
    window_range(g, pos, z, j0, j1);
    const int64_t* pages = g.block_ptrs + g.cu_blocks[s];
    const size_t k_row = (size_t)G * D, v_row = (size_t)G * V;
    for (int jt = j0; jt < j1; jt += kWinTile) {
        const int kt = min(kWinTile, j1 - jt);
        // final softmax weights of every head for the tile's keys: one (key, key/value head) pair per thread
        for (int item = tid; item < kt * G; item += nt) {
            const int c = item / kt, jj = item % kt, j = jt + jj;
            const T* key = reinterpret_cast<const T*>(window_page(g, pages, j)) + (size_t)(j % g.block_len) * k_row + (size_t)c * D;
            for (int hb = 0; hb < rep; hb += kMaxRep) {
                const int cnt = min(kMaxRep, rep - hb);
                float acc[kMaxRep];
                key_dots<T, VEC>(key, qs + (size_t)(c * rep + hb) * D, D, cnt, acc);
#pragma unroll
                for (int u = 0; u < kMaxRep; ++u) {
                    if (u < cnt) {
                        const int h = c * rep + hb + u;
                        p[h * kWinTile + jj] = expf(window_score(g, acc[u], h, pos - j) - mx[h]) * linv[h];
                    }
                }
            }
        }
        __syncthreads();
        if (g.talk) {
            for (int item = tid; item < H * kt; item += nt) {
                const int h = item / kt, jj = item % kt;
                float a = 0.f;
                for (int k = 0; k < H; ++k) a = fmaf(talk[h * H + k], p[k * kWinTile + jj], a);
                p2[h * kWinTile + jj] = a;
            }
            __syncthreads();
        }
        // weighted value sums: one (key/value head, value column) pair per thread, each value read once for the heads that share it
        for (int item = tid; item < G * V; item += nt) {
            const int c = item / V, col = item % V;
            for (int hb = 0; hb < rep; hb += kMaxRep) {
                const int cnt = min(kMaxRep, rep - hb);
                float acc[kMaxRep];
#pragma unroll
                for (int u = 0; u < kMaxRep; ++u) acc[u] = 0.f;
                for (int jj = 0; jj < kt; ++jj) {
                    const int j = jt + jj;
                    const T* val = reinterpret_cast<const T*>(window_page(g, pages, j) + g.v_off) + (size_t)(j % g.block_len) * v_row;
                    const float vv = to_f(val[(size_t)c * V + col]);
#pragma unroll
                    for (int u = 0; u < kMaxRep; ++u)
                        if (u < cnt) acc[u] = fmaf(p2[(c * rep + hb + u) * kWinTile + jj], vv, acc[u]);
                }
#pragma unroll
                for (int u = 0; u < kMaxRep; ++u)
                    if (u < cnt) o[(size_t)(c * rep + hb + u) * V + col] += acc[u];
            }
        }
        __syncthreads();
    }
    float* dst = o_part + ((size_t)t * g.splits + z) * H * V;
    for (int i = tid; i < H * V; i += nt) dst[i] = o[i];
}

// y[t, i] = (sum over ranges of o_part[t, z, i]) * sigmoid(gate[t, i]) as T
template <typename T>
__global__ void window_out_kernel(const float* __restrict__ o_part, int splits, int cols, const T* __restrict__ gate, int64_t ld_gate,
                                  T* __restrict__ y)
{
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float a = 0.f;
        for (int z = 0; z < splits; ++z) a += o_part[((size_t)t * splits + z) * cols + i];
        if (gate) a *= sigmoid_f(to_f(gate[(size_t)t * ld_gate + i]));
        y[(size_t)t * cols + i] = from_f<T>(a);
    }
}
