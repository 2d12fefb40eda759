// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16 with
// float32 accumulation), for head sizes 16..128 in steps of 16. Same contracts and the
// same math as the generic kernels in attention.cu (scores, softmax and the weighted sum
// accumulate in float32; causal mask with an optional window), which stay in use for
// float32 and for larger heads.
//
//   decode:  a block owns (request, key head, split of the keys). The query heads that
//            share the key head are the rows of one 16-row tile, so one pass over the
//            keys serves them all. Each of the 4 warps streams its own 16-key tiles
//            through a 3-stage cp.async pipeline; the warps' partial results are merged
//            in shared memory into one (max, sum, weighted values) record per head. Up
//            to 16 splits of a (request, key head) run as one thread-block cluster and
//            merge there: every block sends its records into the shared memory of the
//            block that merges that part of the output. More splits write their records
//            to global memory, and the combine kernel of attention.cu merges them.
//   prefill: a block owns (64 query tokens of one request, query head); 4 warps of 16
//            rows; keys and values come in tiles of 64 through a double buffer.
#include <mutex>

#include "common.cuh"
#include "mma_util.cuh"

typedef __nv_bfloat16 bf16;

constexpr float LOG2E = 1.4426950408889634f;

// 2^x on the special-function unit (2 ulp; 2^-inf = 0). The softmax works in the log2 domain:
// exp(s * scale - m) = 2^(s * scale * log2(e) - m'), one FMA and one ex2 per score.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------
// Decode
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void dm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float dm_ld_cluster(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ void dm_st_cluster(uint32_t local_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void dm_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void dm_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

constexpr int DM_WARPS = 4, DM_THREADS = DM_WARPS * 32, DM_STAGES = 3, DM_TILE = 16;

// Shared memory of the decode kernel: the warps' rings of tiles (re-used for their merge), and behind them,
// when the splits merge as a cluster, what the other blocks send: per sender the maximum and the sum of each
// of the ng heads, and this block's share of the ng * d outputs (dealt out in runs of 32 over the blocks).
constexpr int DM_STAGES_LIGHT = 2;   // the ring of the kernel of which three blocks fit an SM (see the kernel)
__host__ __device__ constexpr size_t dm_ring_bytes(int d, int stages = DM_STAGES) {
  const size_t pipe = (size_t)DM_WARPS * stages * 2 * DM_TILE * (d + 8) * 2;
  const size_t merge = (size_t)(DM_WARPS * 16 * d + 2 * DM_WARPS * 16 + 16 * (d + 2)) * 4;
  return ((pipe > merge ? pipe : merge) + 15) / 16 * 16;
}
__host__ __device__ inline int dm_share(int ng, int d, int splits) {   // outputs a block merges, a multiple of 32
  return (ng * d + 32 * splits - 1) / (32 * splits) * 32;
}
__host__ __device__ inline size_t dm_inbox_bytes(int ng, int d, int splits) {
  return (size_t)splits * (2 * ng + dm_share(ng, d, splits)) * 4;
}

// SWAP (at most 8 query heads per key head, the usual case): the keys are the 16 rows of the MMA and the heads its
// 8 columns (S^T = K Q^T, O^T = V^T P^T), so a tile of 16 keys takes one MMA per 16 elements of the head where the
// other orientation (heads on the 16 rows, most of them padding) takes two; P goes from the accumulators' layout
// to the operand's by a transposing register move (movmatrix). The legacy tensor path is slow enough on this part
// that the MMAs of a tile are a large part of a warp's time per tile.
// STAGES: tiles of a warp's ring. Three: two tiles on their way while one is used, two blocks an SM. Two (head_dim
// 128, keys on the MMA's rows only): one tile on its way, three blocks an SM: slower when either fits the step's
// blocks in one wave (4.13 against 3.58 ms a step at 32 requests with contexts of 512), faster when only it does
// (40 requests: 4.07 against 4.97 ms), so the caller asks for it per launch (llmrs_attn_decode_next_ring).
template <int DCH, bool SWAP, int STAGES = DM_STAGES>
__global__ void __launch_bounds__(DM_THREADS)
attn_decode_split_mma_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ cache,
                             const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                             const int* __restrict__ cached_len, const int* __restrict__ block_table,
                             int table_stride, float* __restrict__ part, int max_splits, int split_keys,
                             int n_q_heads, int n_kv_heads, int page_size, int window, float scale,
                             bf16* __restrict__ out, long long out_stride, int* __restrict__ counters,
                             int cluster_merge, const L2Prefetch next) {
  constexpr int D = 16 * DCH;
  constexpr int ROW = D + 8;               // 16 bytes of padding: ldmatrix rows fall into distinct banks
  constexpr int CH = D / 8;                // 16-byte chunks per row
  constexpr int TILE_ELEMS = DM_TILE * ROW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  // A block may write into another's shared memory only once that block runs: every block of the cluster
  // says so here, and waits for the others just before its first such write.
  if (cluster_merge) dm_cluster_arrive();
  // Up to the wait below only data of earlier steps is read: the step's index arrays and
  // cached keys and values other than the newest position (the only one written in this step).

  const int G = n_q_heads / n_kv_heads;
  const int hgroups = (G + 15) / 16;
  const int di = blockIdx.x;
  const int kvh = blockIdx.y / hgroups;
  const int g0 = (blockIdx.y % hgroups) * 16;
  const int ng = min(16, G - g0);
  const int split = blockIdx.z;
  const int req = dec_reqs[di];
  const int kv_len = cached_len[req] + 1;
  const int kv_lo = window > 0 ? max(0, kv_len - window) : 0;
  const int k_begin = max(split * split_keys, kv_lo);
  const int k_end = min((split + 1) * split_keys, kv_len);
  // A split without keys has nothing to do, but as a member of a cluster that merges the splits it
  // still has to meet the others at the cluster's barriers (with an empty record).
  const bool empty = k_begin >= k_end;
  if (empty && !cluster_merge) return;
  const int* table = block_table + (size_t)req * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;

  const int tile_first = k_begin / DM_TILE, tile_last = empty ? tile_first - 1 : (k_end - 1) / DM_TILE;
  const int n_tiles = tile_last - tile_first + 1;
  const int n_my = n_tiles > warp ? (n_tiles - warp + DM_WARPS - 1) / DM_WARPS : 0;

  bf16* wbase = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * STAGES * 2 * TILE_ELEMS;

  // When a page holds whole 16-key tiles, a tile is one contiguous run of rows in one
  // page: lane j keeps the page of the warp's j-th tile (of the current 32), so the
  // copies need neither a table look-up nor a division on their way out.
  const bool page_tiles = page_size % DM_TILE == 0;
  int my_pages = 0, pages_base = -1;
  auto load_tile = [&](int i, int stage) {
    const int t = tile_first + warp + i * DM_WARPS;
    bf16* Ks = wbase + (size_t)stage * 2 * TILE_ELEMS;
    bf16* Vs = Ks + TILE_ELEMS;
    if (page_tiles) {
      if ((i >> 5) != pages_base) {
        pages_base = i >> 5;
        const int ti = tile_first + warp + ((pages_base << 5) + lane) * DM_WARPS;
        my_pages = ti <= tile_last ? LLMRS_CHECKED_PAGE(table[(ti * DM_TILE) / page_size], 4, ti * DM_TILE) : 0;
      }
      const int page = __shfl_sync(0xffffffffu, my_pages, i & 31);
      const bf16* kbase = cache + kv_tile_offset(page, kvh, 0, n_kv_heads, page_size, D) +
                          (size_t)((t * DM_TILE) % page_size) * D;
      const bf16* vbase = kbase + (size_t)page_size * D;
      const int key0 = t * DM_TILE;
      if (key0 >= k_begin && key0 + DM_TILE <= k_end) {
        // Whole tile inside the split: 16 rows of K are one contiguous run, so are the 16 rows of V.
#pragma unroll
        for (int j = 0; j < (DM_TILE * CH + 31) / 32; ++j) {
          const int c = lane + 32 * j;
          if ((DM_TILE * CH) % 32 == 0 || c < DM_TILE * CH) {
            const int row = c / CH, ch = c - row * CH;
            cp_async_16(Ks + row * ROW + ch * 8, kbase + c * 8, 16);
            cp_async_16(Vs + row * ROW + ch * 8, vbase + c * 8, 16);
          }
        }
        return;
      }
#pragma unroll 4
      for (int c = lane; c < DM_TILE * CH; c += 32) {
        const int row = c / CH, ch = c - row * CH;
        const bool valid = key0 + row >= k_begin && key0 + row < k_end;
        cp_async_16(Ks + row * ROW + ch * 8, valid ? kbase + c * 8 : cache, valid ? 16 : 0);
        cp_async_16(Vs + row * ROW + ch * 8, valid ? vbase + c * 8 : cache, valid ? 16 : 0);
      }
      return;
    }
#pragma unroll 4
    for (int c = lane; c < DM_TILE * CH; c += 32) {
      const int row = c / CH, ch = c - row * CH;
      const int key = t * DM_TILE + row;
      const bool valid = key >= k_begin && key < k_end;
      const bf16* src = cache;
      if (valid) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 4, key);
        src = cache + kv_tile_offset(page, kvh, 0, n_kv_heads, page_size, D) + (size_t)(key % page_size) * D + ch * 8;
      }
      cp_async_16(Ks + row * ROW + ch * 8, src, valid ? 16 : 0);
      cp_async_16(Vs + row * ROW + ch * 8, valid ? src + (size_t)page_size * D : src, valid ? 16 : 0);
    }
  };

  float o[2 * DCH][4];
#pragma unroll
  for (int n = 0; n < 2 * DCH; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  const float sl2 = scale * LOG2E;

  // Accumulators of the swapped orientation: O^T per 16 elements of the head (rows) and the heads 2tq, 2tq+1
  // (columns); the running maximum and sum of those two heads (the same in the eight lanes that share tq).
  float ot[DCH][4];
#pragma unroll
  for (int n = 0; n < DCH; ++n) ot[n][0] = ot[n][1] = ot[n][2] = ot[n][3] = 0.f;
  float m_h[2] = {-INFINITY, -INFINITY}, l_h[2] = {0.f, 0.f};
  // The first tiles are requested before the wait on the preceding kernels (they overlap
  // those kernels' tails), except a tile that holds the newest key, which this step writes.
  const int new_tile = (kv_len - 1) / DM_TILE;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_my && tile_first + warp + s * DM_WARPS < new_tile) load_tile(s, s);
    cp_async_commit();
  }
  pdl_wait();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_my && tile_first + warp + s * DM_WARPS >= new_tile) load_tile(s, s);
    cp_async_commit();
  }
  if constexpr (SWAP) {
    // Q^T as B fragments (k = element of the head, n = head): lane (gq, tq) holds elements 2tq, 2tq+1 (and +8) of
    // head gq for every 16 elements; heads beyond the group are zero.
    uint32_t qb[DCH][2];
    {
      const bf16* qh = q + (size_t)q_start[req] * q_stride + (size_t)(kvh * G + g0 + gq) * D;
#pragma unroll
      for (int kc = 0; kc < DCH; ++kc) {
        qb[kc][0] = gq < ng ? *reinterpret_cast<const uint32_t*>(qh + kc * 16 + tq * 2) : 0u;
        qb[kc][1] = gq < ng ? *reinterpret_cast<const uint32_t*>(qh + kc * 16 + tq * 2 + 8) : 0u;
      }
    }
    for (int i = 0; i < n_my; ++i) {
      cp_async_wait<STAGES - 2>();
      __syncwarp();
      if (i + STAGES - 1 < n_my) load_tile(i + STAGES - 1, (i + STAGES - 1) % STAGES);
      cp_async_commit();

      const bf16* Ks = wbase + (size_t)(i % STAGES) * 2 * TILE_ELEMS;
      const bf16* Vs = Ks + TILE_ELEMS;
      const int key0 = (tile_first + warp + i * DM_WARPS) * DM_TILE;
      const int j = lane >> 3;

      // S^T: 16 keys (rows) x 8 heads (columns). s[0], s[1]: key gq, heads 2tq, 2tq+1; s[2], s[3]: key gq + 8.
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kc = 0; kc < DCH; ++kc) {
        uint32_t a[4];
        // matrix j: keys (j%2)*8.., elements of the head kc*16 + (j/2)*8..
        ldmatrix_x4(a, Ks + ((j & 1) * 8 + (lane & 7)) * ROW + kc * 16 + (j >> 1) * 8);
        mma_bf16_16816(sc, a, qb[kc][0], qb[kc][1]);
      }
      const bool edge = key0 < k_begin || key0 + DM_TILE > k_end;
      if (edge) {
        const bool seen_lo = key0 + gq >= k_begin && key0 + gq < k_end;
        const bool seen_hi = key0 + gq + 8 >= k_begin && key0 + gq + 8 < k_end;
        sc[0] = seen_lo ? sc[0] : -INFINITY; sc[1] = seen_lo ? sc[1] : -INFINITY;
        sc[2] = seen_hi ? sc[2] : -INFINITY; sc[3] = seen_hi ? sc[3] : -INFINITY;
      }
      float corr[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {       // this lane's two heads; the keys of a head are spread over gq
        float mx = fmaxf(sc[h], sc[2 + h]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_h[h], mx * sl2);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = ex2(m_h[h] - m_use);
        m_h[h] = m_new;
        const float p0 = ex2(fmaf(sc[h], sl2, -m_use)), p1 = ex2(fmaf(sc[2 + h], sl2, -m_use));
        sc[h] = p0;
        sc[2 + h] = p1;
        float sum = p0 + p1;
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        l_h[h] = l_h[h] * corr[h] + sum;
      }
      // P^T as B fragments (k = key, n = head): the accumulators hold (key gq, heads 2tq..), the operand wants
      // (keys 2tq.., head gq): one transposing move per 8 keys.
      uint32_t pb0, pb1;
      {
        const uint32_t lo = pack_bf16(sc[0], sc[1]), hi = pack_bf16(sc[2], sc[3]);
        asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(lo));
        asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(hi));
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int n = 0; n < DCH; ++n) {
          ot[n][0] *= corr[0]; ot[n][1] *= corr[1]; ot[n][2] *= corr[0]; ot[n][3] *= corr[1];
        }
      }
      // O^T += V^T P^T: rows are 16 elements of the head, the A fragments are 8x8 blocks of V read transposed.
#pragma unroll
      for (int nc = 0; nc < DCH; ++nc) {
        uint32_t a[4];
        // matrix j: keys (j/2)*8.., elements of the head nc*16 + (j%2)*8..
        ldmatrix_x4_trans(a, Vs + ((j >> 1) * 8 + (lane & 7)) * ROW + nc * 16 + (j & 1) * 8);
        mma_bf16_16816(ot[nc], a, pb0, pb1);
      }
    }
  } else {
  // Query rows as A fragments: row gq is head g0+gq, row gq+8 is head g0+gq+8; absent heads are zero.
  uint32_t qf[DCH][4];
  {
    const bf16* qt = q + (size_t)q_start[req] * q_stride + (size_t)(kvh * G + g0) * D;
#pragma unroll
    for (int kc = 0; kc < DCH; ++kc) {
      const int col = kc * 16 + tq * 2;
      qf[kc][0] = gq < ng ? *reinterpret_cast<const uint32_t*>(qt + (size_t)gq * D + col) : 0u;
      qf[kc][1] = gq + 8 < ng ? *reinterpret_cast<const uint32_t*>(qt + (size_t)(gq + 8) * D + col) : 0u;
      qf[kc][2] = gq < ng ? *reinterpret_cast<const uint32_t*>(qt + (size_t)gq * D + col + 8) : 0u;
      qf[kc][3] = gq + 8 < ng ? *reinterpret_cast<const uint32_t*>(qt + (size_t)(gq + 8) * D + col + 8) : 0u;
    }
  }
  // The ring was filled with 2 * (STAGES - 1) groups: tile s (s < STAGES - 1) lies in group
  // s or STAGES - 1 + s, tile i >= STAGES - 1 in group STAGES - 1 + i. Leaving the newest
  // STAGES - 2 groups pending at iteration i still covers tile i.
  for (int i = 0; i < n_my; ++i) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (i + STAGES - 1 < n_my) load_tile(i + STAGES - 1, (i + STAGES - 1) % STAGES);
    cp_async_commit();

    const bf16* Ks = wbase + (size_t)(i % STAGES) * 2 * TILE_ELEMS;
    const bf16* Vs = Ks + TILE_ELEMS;
    const int key0 = (tile_first + warp + i * DM_WARPS) * DM_TILE;

    // Scores of the 16 head rows against 16 keys: two 16x8 tiles.
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kc = 0; kc < DCH; ++kc) {
      uint32_t b[4];
      // matrix j = lane/8: keys (j/2)*8.., head-dim columns kc*16 + (j%2)*8..
      const int j = lane >> 3;
      ldmatrix_x4(b, Ks + ((j >> 1) * 8 + (lane & 7)) * ROW + kc * 16 + (j & 1) * 8);
      mma_bf16_16816(s[0], qf[kc], b[0], b[1]);
      mma_bf16_16816(s[1], qf[kc], b[2], b[3]);
    }
    // Mask (only a tile on the split's edge has keys to hide), scale into the log2 domain,
    // online softmax per row.
    float mx[2] = {-INFINITY, -INFINITY};
    const bool edge = key0 < k_begin || key0 + DM_TILE > k_end;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + n * 8 + tq * 2 + (e & 1);
        const bool seen = !edge || (key >= k_begin && key < k_end);
        s[n][e] = seen ? s[n][e] : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
    uint32_t pf[4];
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_row[r], mx[r] * sl2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = ex2(m_row[r] - m_use);
      m_row[r] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float p = ex2(fmaf(s[n][r * 2 + e], sl2, -m_use));
          s[n][r * 2 + e] = p;
          sum += p;
        }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_row[r] = l_row[r] * corr[r] + sum;
    }
    pf[0] = pack_bf16(s[0][0], s[0][1]);
    pf[1] = pack_bf16(s[0][2], s[0][3]);
    pf[2] = pack_bf16(s[1][0], s[1][1]);
    pf[3] = pack_bf16(s[1][2], s[1][3]);
    // The running maximum seldom moves after the first tiles: rescale only when some row's did.
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int n = 0; n < 2 * DCH; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
    // Weighted sum of values: B fragments are 8x8 blocks of V read transposed.
#pragma unroll
    for (int nc = 0; nc < DCH; ++nc) {
      uint32_t b[4];
      // matrix j = lane/8: keys (j%2)*8.., head-dim columns (2*nc + j/2)*8..
      const int j = lane >> 3;
      ldmatrix_x4_trans(b, Vs + ((j & 1) * 8 + (lane & 7)) * ROW + (2 * nc + (j >> 1)) * 8);
      mma_bf16_16816(o[2 * nc], pf, b[0], b[1]);
      mma_bf16_16816(o[2 * nc + 1], pf, b[2], b[3]);
    }
  }
  }
  // The block's last keys and values are on their way: the weights of the product that follows attention
  // (see L2Prefetch) can come into the L2 while this block merges its warps and its cluster.
  if (threadIdx.x == 0) l2_prefetch_slice(next);
  cp_async_wait<0>();
  __syncthreads();

  // Merge the warps: every warp leaves (m, l, o) of its rows in shared memory.
  float* Om = reinterpret_cast<float*>(smem_raw);           // [warps][16][D]
  float* Mm = Om + DM_WARPS * 16 * D;                       // [warps][16]
  float* Lm = Mm + DM_WARPS * 16;
  if constexpr (SWAP) {
    // Rows of Om are heads (2tq, 2tq+1 of this lane), columns elements of the head (gq and gq + 8 of every 16).
#pragma unroll
    for (int n = 0; n < DCH; ++n) {
      float* h0 = Om + ((size_t)warp * 16 + tq * 2) * D + n * 16 + gq;
      float* h1 = h0 + D;
      h0[0] = ot[n][0]; h1[0] = ot[n][1]; h0[8] = ot[n][2]; h1[8] = ot[n][3];
    }
    if (gq == 0) {
      Mm[warp * 16 + tq * 2] = m_h[0]; Mm[warp * 16 + tq * 2 + 1] = m_h[1];
      Lm[warp * 16 + tq * 2] = l_h[0]; Lm[warp * 16 + tq * 2 + 1] = l_h[1];
    }
  } else {
#pragma unroll
    for (int n = 0; n < 2 * DCH; ++n) {
      const int col = n * 8 + tq * 2;
      float* r0 = Om + ((size_t)warp * 16 + gq) * D + col;
      float* r1 = Om + ((size_t)warp * 16 + gq + 8) * D + col;
      r0[0] = o[n][0]; r0[1] = o[n][1]; r1[0] = o[n][2]; r1[1] = o[n][3];
    }
    if (tq == 0) {
      Mm[warp * 16 + gq] = m_row[0]; Mm[warp * 16 + gq + 8] = m_row[1];
      Lm[warp * 16 + gq] = l_row[0]; Lm[warp * 16 + gq + 8] = l_row[1];
    }
  }
  __syncthreads();
  const int S = (int)gridDim.z;
  const int share = dm_share(ng, D, S);
  float* inbox_ml = reinterpret_cast<float*>(smem_raw + dm_ring_bytes(D, STAGES));   // [S][ng][2]
  float* inbox_o = inbox_ml + (size_t)S * ng * 2;                            // [S][share]
  if (cluster_merge) dm_cluster_wait();   // every block of the cluster runs
  for (int i = threadIdx.x; i < ng * D; i += DM_THREADS) {
    const int g = i / D, e = i - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) M = fmaxf(M, Mm[w * 16 + g]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float mw = Mm[w * 16 + g];
      const float f = mw == -INFINITY ? 0.f : ex2(mw - M);
      L += Lm[w * 16 + g] * f;
      acc += Om[((size_t)w * 16 + g) * D + e] * f;
    }
    const int head = kvh * G + g0 + g;
    if (cluster_merge) {
      // The splits of a (request, key head) are the blocks of one cluster. Output i goes to the block that
      // merges it (runs of 32 outputs go round the blocks), each head's maximum and sum to all of them.
      const int run = i >> 5;
      dm_st_cluster((uint32_t)__cvta_generic_to_shared(inbox_o + (size_t)split * share + (run / S) * 32 + (i & 31)),
                    (uint32_t)(run % S), acc);
      if (e == 0) {
        const uint32_t ml = (uint32_t)__cvta_generic_to_shared(inbox_ml + ((size_t)split * ng + g) * 2);
        for (int r = 0; r < S; ++r) {
          dm_st_cluster(ml, (uint32_t)r, M);
          dm_st_cluster(ml + 4, (uint32_t)r, L);
        }
      }
      continue;
    }
    float* pp = part + ((size_t)((size_t)di * n_q_heads + head) * max_splits + split) * (D + 2);
    pp[2 + e] = acc;
    // The combine step works with natural logarithms: hand it the maximum in that domain.
    if (e == 0) { pp[0] = M / LOG2E; pp[1] = L; }
  }
  if (cluster_merge) {
    // After the cluster's barrier every block holds what the others sent it and merges its share: no pass
    // through global memory, no second kernel, and nobody reads another block's memory, so a block may
    // leave as soon as it is done.
    dm_cluster_arrive();
    dm_cluster_wait();
    for (int s = (int)threadIdx.x; s < share; s += DM_THREADS) {
      const int i = ((s >> 5) * S + split) * 32 + (s & 31);
      if (i >= ng * D) continue;
      const int g = i / D, e = i - g * D;
      float M = -INFINITY;
      for (int r = 0; r < S; ++r) M = fmaxf(M, inbox_ml[((size_t)r * ng + g) * 2]);
      float L = 0.f, a = 0.f;
      for (int r = 0; r < S; ++r) {
        const float mr = inbox_ml[((size_t)r * ng + g) * 2];
        const float f = mr == -INFINITY ? 0.f : ex2(mr - M);
        L += inbox_ml[((size_t)r * ng + g) * 2 + 1] * f;
        a += inbox_o[(size_t)r * share + s] * f;
      }
      out[(size_t)q_start[req] * out_stride + (size_t)(kvh * G + g0 + g) * D + e] = __float2bfloat16_rn(a / L);
    }
    return;
  }
  if (counters == nullptr) return;   // a separate kernel merges the splits

  // The block that finishes last for its (request, head group) merges the splits itself:
  // a counter per group is raised by every block after its records are visible, and put
  // back to zero by the one that sees the full count.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  const int s_first = kv_lo / split_keys, s_last = (kv_len - 1) / split_keys;
  if (threadIdx.x == 0) {
    int* c = counters + (size_t)di * gridDim.y + blockIdx.y;
    const int seen = atomicAdd(c, 1);
    is_last = seen == s_last - s_first;
    if (is_last) *c = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < ng * D; i += DM_THREADS) {
    const int g = i / D, e = i - g * D;
    const int head = kvh * G + g0 + g;
    const float* base = part + ((size_t)((size_t)di * n_q_heads + head) * max_splits) * (D + 2);
    float m = -INFINITY;
    for (int sp = s_first; sp <= s_last; ++sp) m = fmaxf(m, __ldcg(base + (size_t)sp * (D + 2)));
    float l = 0.f, a = 0.f;
    for (int sp = s_first; sp <= s_last; ++sp) {
      const float* pp = base + (size_t)sp * (D + 2);
      const float f = expf(__ldcg(pp) - m);
      l += __ldcg(pp + 1) * f;
      a += __ldcg(pp + 2 + e) * f;
    }
    out[(size_t)q_start[req] * out_stride + (size_t)head * D + e] = __float2bfloat16_rn(a / l);
  }
}

// Lets the kernel use `smem` bytes of dynamic shared memory and clusters of up to 16 blocks (more than the
// portable 8, for few requests). The limit only ever grows: the launcher and the capacity query below share
// it, and a query for a small cluster must not take away what a launch with a large one was given.
template <int DCH>
static int decode_mma_allow(size_t smem) {
  static size_t allowed = 0;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<DCH, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<DCH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<DCH, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<DCH, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: clusters of 16: %s", cudaGetErrorString(e));
    allowed = smem;
  }
  return 0;
}

// The same for the kernel with the ring of two tiles (head_dim 128, keys on the MMA's rows).
static int decode_mma_allow_light(size_t smem) {
  static size_t allowed = 0;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<8, true, DM_STAGES_LIGHT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    e = cudaFuncSetAttribute(attn_decode_split_mma_kernel<8, true, DM_STAGES_LIGHT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: clusters of 16: %s", cudaGetErrorString(e));
    allowed = smem;
  }
  return 0;
}
static bool decode_mma_light_applies(int dch, int n_q_heads, int n_kv_heads) { return dch == 8 && n_q_heads / n_kv_heads <= 8; }

// The ring of the NEXT launch of the tensor-core decode kernel: 2 asks for the kernel with the ring of two tiles where
// it exists (head_dim 128, at most 8 query heads per key head), anything else for the usual one. One launch takes it.
static int g_next_ring = 0;
LLMRS_API void llmrs_attn_decode_next_ring(int stages) { g_next_ring = stages; }

template <int DCH>
static int launch_decode_mma(const void* q, long long q_stride, const void* cache, const int* dec_reqs, int n_dec,
                             const int* q_start, const int* cached_len, const int* block_table, int table_stride,
                             float* scratch, int max_splits, int split_keys, int n_q_heads, int n_kv_heads,
                             int page_size, int window, float scale, void* out, long long out_stride, int* counters,
                             int cluster_merge, const L2Prefetch& next, cudaStream_t stream) {
  constexpr int D = 16 * DCH;
  const int ng_max = n_q_heads / n_kv_heads < 16 ? n_q_heads / n_kv_heads : 16;
  const bool light = g_next_ring == DM_STAGES_LIGHT && decode_mma_light_applies(DCH, n_q_heads, n_kv_heads);
  g_next_ring = 0;
  const size_t smem = dm_ring_bytes(D, light ? DM_STAGES_LIGHT : DM_STAGES) + (cluster_merge ? dm_inbox_bytes(ng_max, D, max_splits) : 0);
  if (int rc = light ? decode_mma_allow_light(smem) : decode_mma_allow<DCH>(smem)) return rc;
  const int G = n_q_heads / n_kv_heads;
  dim3 grid(n_dec, n_kv_heads * ((G + 15) / 16), max_splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(DM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  if (g_llmrs_pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (cluster_merge) {   // the splits of a (request, key head) form a cluster
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = max_splits;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  // At most eight query heads per key head: the keys take the MMA's rows (see the kernel).
  auto kernel = G <= 8 ? attn_decode_split_mma_kernel<DCH, true> : attn_decode_split_mma_kernel<DCH, false>;
  if constexpr (DCH == 8) {
    if (light) kernel = attn_decode_split_mma_kernel<8, true, DM_STAGES_LIGHT>;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, (const bf16*)q, q_stride, (const bf16*)cache,
                                     dec_reqs, q_start, cached_len, block_table, table_stride, scratch, max_splits,
                                     split_keys, n_q_heads, n_kv_heads, page_size, window, scale, (bf16*)out,
                                     out_stride, counters, cluster_merge, next);
  if (e != cudaSuccess) return llmrs_fail("attn_decode_mma launch: %s", cudaGetErrorString(e));
  return llmrs_launch_status("attn_decode_split_mma");
}

template <int DCH>
static int decode_mma_capacity(int cluster, int ng, int* blocks, bool light = false) {
  constexpr int D = 16 * DCH;
  const size_t smem = dm_ring_bytes(D, light ? DM_STAGES_LIGHT : DM_STAGES) + (cluster > 1 ? dm_inbox_bytes(ng, D, cluster) : 0);
  if (int rc = light ? decode_mma_allow_light(smem) : decode_mma_allow<DCH>(smem)) return rc;
  cudaError_t e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(64, 8, cluster);
  cfg.blockDim = dim3(DM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if constexpr (DCH == 8) {
    if (light) {
      e = cudaOccupancyMaxActiveClusters(&n, attn_decode_split_mma_kernel<8, true, DM_STAGES_LIGHT>, &cfg);
      if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: occupancy of clusters of %d: %s", cluster, cudaGetErrorString(e));
      *blocks = n * cluster;
      return 0;
    }
  }
  e = ng <= 8 ? cudaOccupancyMaxActiveClusters(&n, attn_decode_split_mma_kernel<DCH, true>, &cfg)
              : cudaOccupancyMaxActiveClusters(&n, attn_decode_split_mma_kernel<DCH, false>, &cfg);
  if (e != cudaSuccess) return llmrs_fail("attn_decode_mma: occupancy of clusters of %d: %s", cluster, cudaGetErrorString(e));
  *blocks = n * cluster;
  return 0;
}

// How many blocks of the tensor-core decode kernel the device holds at a time when they come in clusters
// of `cluster` (1 to 16) and serve `ng` query heads (1 to 16) per key head: what the caller needs to cut the
// keys so that a step's blocks fill whole waves.
LLMRS_API int llmrs_attn_decode_capacity(int d, int cluster, int ng, int* blocks) {
  if (cluster < 1 || cluster > 16 || ng < 1 || ng > 16 || d % 16 || d < 16 || d > 128)
    return llmrs_fail("attn_decode_capacity: head_dim %d, clusters of %d, %d heads", d, cluster, ng);
  switch (d / 16) {
    case 1: return decode_mma_capacity<1>(cluster, ng, blocks);
    case 2: return decode_mma_capacity<2>(cluster, ng, blocks);
    case 3: return decode_mma_capacity<3>(cluster, ng, blocks);
    case 4: return decode_mma_capacity<4>(cluster, ng, blocks);
    case 5: return decode_mma_capacity<5>(cluster, ng, blocks);
    case 6: return decode_mma_capacity<6>(cluster, ng, blocks);
    case 7: return decode_mma_capacity<7>(cluster, ng, blocks);
    default: return decode_mma_capacity<8>(cluster, ng, blocks);
  }
}

// The same for the kernel with the ring of two tiles; *blocks = 0 where that kernel does not exist (head_dim other than
// 128, more than 8 query heads per key head).
LLMRS_API int llmrs_attn_decode_capacity_light(int d, int cluster, int ng, int* blocks) {
  if (cluster < 1 || cluster > 16 || ng < 1 || ng > 16 || d % 16 || d < 16 || d > 128)
    return llmrs_fail("attn_decode_capacity: head_dim %d, clusters of %d, %d heads", d, cluster, ng);
  *blocks = 0;
  if (!decode_mma_light_applies(d / 16, ng, 1)) return 0;
  return decode_mma_capacity<8>(cluster, ng, blocks, true);
}

// The split step of decode attention on the tensor cores (bfloat16, head_dim <= 128).
// Writes the same per-split records as the generic split kernel. With `counters` (zeroed ints, one per
// request and head group; the kernel leaves them zero) the last block of each group also merges the
// splits into `out`; with `cluster_merge` (max_splits <= 16) the splits of a group run as one cluster and
// merge through distributed shared memory; else the caller runs the combine kernel.
int llmrs_attn_decode_split_mma(const void* q, long long q_stride, const void* cache, const int* dec_reqs, int n_dec,
                                const int* q_start, const int* cached_len, const int* block_table, int table_stride,
                                float* scratch, int max_splits, int split_keys, int n_q_heads, int n_kv_heads, int d,
                                int page_size, int window, float scale, void* out, long long out_stride,
                                int* counters, int cluster_merge, const L2Prefetch& next, cudaStream_t stream) {
  if (cluster_merge && (max_splits < 1 || max_splits > 16))
    return llmrs_fail("attn_decode_mma: a cluster merges at most 16 splits, got %d", max_splits);
#define LLMRS_DM_CASE(N)                                                                                          \
  case N:                                                                                                          \
    return launch_decode_mma<N>(q, q_stride, cache, dec_reqs, n_dec, q_start, cached_len, block_table, table_stride, \
                                scratch, max_splits, split_keys, n_q_heads, n_kv_heads, page_size, window, scale, out, \
                                out_stride, counters, cluster_merge, next, stream)
  switch (d / 16) {
    LLMRS_DM_CASE(1); LLMRS_DM_CASE(2); LLMRS_DM_CASE(3); LLMRS_DM_CASE(4);
    LLMRS_DM_CASE(5); LLMRS_DM_CASE(6); LLMRS_DM_CASE(7); LLMRS_DM_CASE(8);
  }
#undef LLMRS_DM_CASE
  return llmrs_fail("attn_decode_mma: head_dim %d is not supported", d);
}

// ---------------------------------------------------------------------------------
// Prefill
// ---------------------------------------------------------------------------------
constexpr int PM_BQ = 64, PM_BK = 64, PM_WARPS = 4, PM_THREADS = PM_WARPS * 32;

template <int DCH>
__global__ void __launch_bounds__(PM_THREADS, 3)
attn_prefill_mma_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                        const bf16* __restrict__ cache, const int* __restrict__ tiles,
                        const int* __restrict__ q_start, const int* __restrict__ n_new,
                        const int* __restrict__ cached_len, const int* __restrict__ block_table, int table_stride,
                        int n_q_heads, int n_kv_heads, int page_size, int window, float scale) {
  constexpr int D = 16 * DCH;
  constexpr int ROW = D + 8;
  constexpr int CH = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* KV = reinterpret_cast<bf16*>(smem_raw);     // 2 stages x (K [64][ROW], V [64][ROW])

  // Blocks start in the order of blockIdx.x: all heads of the last tile first (a later tile of a
  // prompt sees more keys), so that the long blocks do not end the kernel alone.
  const int head = blockIdx.x % n_q_heads;
  const int tile = (int)(gridDim.x / n_q_heads) - 1 - (int)(blockIdx.x / n_q_heads);
  const int kvh = head / (n_q_heads / n_kv_heads);
  const int req = tiles[2 * tile], q_off = tiles[2 * tile + 1];
  const int rows = min(PM_BQ, n_new[req] - q_off);
  const int tok0 = q_start[req] + q_off;
  const int pos0 = cached_len[req] + q_off;
  const int kv_hi = pos0 + rows;
  int kv_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  kv_lo = (kv_lo / PM_BK) * PM_BK;
  const int key_floor = window > 0 ? max(0, pos0 - window + 1) : 0;   // no row reads a key below this
  const int* table = block_table + (size_t)req * table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;

  auto load_kv = [&](int kb, int stage) {
    bf16* Ks = KV + (size_t)stage * 2 * PM_BK * ROW;
    bf16* Vs = Ks + PM_BK * ROW;
    for (int c = threadIdx.x; c < PM_BK * CH; c += PM_THREADS) {
      const int row = c / CH, ch = c - row * CH;
      const int key = kb + row;
      const bool valid = key >= key_floor && key < kv_hi;
      const bf16* src = cache;
      if (valid) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 4, key);
        src = cache + kv_tile_offset(page, kvh, 0, n_kv_heads, page_size, D) + (size_t)(key % page_size) * D + ch * 8;
      }
      cp_async_16(Ks + row * ROW + ch * 8, src, valid ? 16 : 0);
      cp_async_16(Vs + row * ROW + ch * 8, valid ? src + (size_t)page_size * D : src, valid ? 16 : 0);
    }
  };
  load_kv(kv_lo, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // Query rows of this warp as A fragments, straight from global memory (read once).
  uint32_t qf[DCH][4];
  {
    const int r0 = warp * 16 + gq, r1 = r0 + 8;
    const bf16* q0 = q + (size_t)(tok0 + r0) * q_stride + (size_t)head * D;
    const bf16* q1 = q + (size_t)(tok0 + r1) * q_stride + (size_t)head * D;
#pragma unroll
    for (int kc = 0; kc < DCH; ++kc) {
      const int col = kc * 16 + tq * 2;
      qf[kc][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
      qf[kc][1] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
      qf[kc][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
      qf[kc][3] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
    }
  }
  float o[2 * DCH][4];
#pragma unroll
  for (int n = 0; n < 2 * DCH; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  const float sl2 = scale * LOG2E;
  const int pos_r[2] = {pos0 + warp * 16 + gq, pos0 + warp * 16 + gq + 8};

  int stage = 0;
  for (int kb = kv_lo; kb < kv_hi; kb += PM_BK, stage ^= 1) {
    // Tile kb is in `stage` (waited for below or before the loop); fetch the next one.
    if (kb + PM_BK < kv_hi) load_kv(kb + PM_BK, stage ^ 1);
    cp_async_commit();
    const bf16* Ks = KV + (size_t)stage * 2 * PM_BK * ROW;
    const bf16* Vs = Ks + PM_BK * ROW;
    // A warp whose rows all lie before this tile of keys has nothing to add.
    const bool active = kb <= pos0 + warp * 16 + 15;
    if (active) {
      float s[PM_BK / 8][4];
#pragma unroll
      for (int n = 0; n < PM_BK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int kc = 0; kc < DCH; ++kc) {
        const int j = lane >> 3;
#pragma unroll
        for (int np = 0; np < PM_BK / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, Ks + (np * 16 + (j >> 1) * 8 + (lane & 7)) * ROW + kc * 16 + (j & 1) * 8);
          mma_bf16_16816(s[2 * np], qf[kc], b[0], b[1]);
          mma_bf16_16816(s[2 * np + 1], qf[kc], b[2], b[3]);
        }
      }
      // Only a tile that touches the diagonal (or the window's far edge) has scores to hide.
      const int pw = pos0 + warp * 16;
      const bool need_mask = kb + PM_BK - 1 > pw || (window > 0 && kb <= pw + 15 - window);
      float mx[2] = {-INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int n = 0; n < PM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb + n * 8 + tq * 2 + (e & 1);
            const int p = pos_r[e >> 1];
            const bool seen = key <= p && (window <= 0 || key > p - window);
            s[n][e] = seen ? s[n][e] : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
          }
      } else {
#pragma unroll
        for (int n = 0; n < PM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_row[r], mx[r] * sl2);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = ex2(m_row[r] - m_use);
        m_row[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < PM_BK / 8; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float p = ex2(fmaf(s[n][r * 2 + e], sl2, -m_use));
            s[n][r * 2 + e] = p;
            sum += p;
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_row[r] = l_row[r] * corr[r] + sum;
      }
#pragma unroll
      for (int n = 0; n < 2 * DCH; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
#pragma unroll
      for (int kc = 0; kc < PM_BK / 16; ++kc) {
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
        pf[1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
        pf[2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
        pf[3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
        const int j = lane >> 3;
#pragma unroll
        for (int nc = 0; nc < DCH; ++nc) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, Vs + (kc * 16 + (j & 1) * 8 + (lane & 7)) * ROW + (2 * nc + (j >> 1)) * 8);
          mma_bf16_16816(o[2 * nc], pf, b[0], b[1]);
          mma_bf16_16816(o[2 * nc + 1], pf, b[2], b[3]);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + gq + r * 8;
    if (row < rows) {
      const float inv = l_row[r] > 0.f ? 1.0f / l_row[r] : 0.f;
      bf16* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)head * D;
#pragma unroll
      for (int n = 0; n < 2 * DCH; ++n) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(o[n][r * 2] * inv, o[n][r * 2 + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(orow + n * 8 + tq * 2) = v;
      }
    }
  }
}

template <int DCH>
static int launch_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* cache,
                              const int* tiles, int n_tiles, const int* q_start, const int* n_new,
                              const int* cached_len, const int* block_table, int table_stride, int n_q_heads,
                              int n_kv_heads, int page_size, int window, float scale, cudaStream_t stream) {
  constexpr int D = 16 * DCH;
  const size_t smem = (size_t)(4 * PM_BK) * (D + 8) * sizeof(bf16);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<DCH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_prefill_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  if ((long long)n_tiles * n_q_heads > 2147483647LL) return llmrs_fail("attn_prefill_mma: %d tiles are too many", n_tiles);
  dim3 grid((unsigned)n_tiles * (unsigned)n_q_heads);
  attn_prefill_mma_kernel<DCH><<<grid, PM_THREADS, smem, stream>>>(
      (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, tiles, q_start, n_new, cached_len,
      block_table, table_stride, n_q_heads, n_kv_heads, page_size, window, scale);
  return llmrs_launch_status("attn_prefill_mma");
}

// Prefill attention on the tensor cores (bfloat16, head_dim <= 128); tiles of 64 queries.
int llmrs_attn_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* cache,
                           const int* tiles, int n_tiles, const int* q_start, const int* n_new,
                           const int* cached_len, const int* block_table, int table_stride, int n_q_heads,
                           int n_kv_heads, int d, int page_size, int window, float scale, cudaStream_t stream) {
#define LLMRS_PM_CASE(N)                                                                                         \
  case N:                                                                                                         \
    return launch_prefill_mma<N>(q, q_stride, out, out_stride, cache, tiles, n_tiles, q_start, n_new, cached_len, \
                                 block_table, table_stride, n_q_heads, n_kv_heads, page_size, window, scale, stream)
  switch (d / 16) {
    LLMRS_PM_CASE(1); LLMRS_PM_CASE(2); LLMRS_PM_CASE(3); LLMRS_PM_CASE(4);
    LLMRS_PM_CASE(5); LLMRS_PM_CASE(6); LLMRS_PM_CASE(7); LLMRS_PM_CASE(8);
  }
#undef LLMRS_PM_CASE
  return llmrs_fail("attn_prefill_mma: head_dim %d is not supported", d);
}
