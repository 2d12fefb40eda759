// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a: operands staged
// in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma issued by
// one thread with the float32 accumulator in tensor memory, read back with tcgen05.ld.
//
//   D[a, b] = sum_k A[a, k] * B[b, k]      A: [a_rows, K], B: [b_rows, K], both K-major
//
// Two ways of mapping a linear layer y = x W^T onto it:
//   mode 0 (many tokens)  A = x (tokens), B = W (features): tile 128 tokens x BN features.
//   mode 1 (few tokens)   A = W (features), B = x (tokens): the 128 rows of the MMA are
//                         filled by weights whatever the batch is, the tokens (16..64) are
//                         the narrow N side. The k range is cut over the blocks of a
//                         thread-block cluster, which add up their partial tiles through
//                         distributed shared memory in a fixed order, so that a skinny
//                         product still puts some hundred blocks on the GPU.
// Epilogues: store (bfloat16 or float32), add into the float32 residual stream,
// SiLU(gate)*up for a weight whose rows alternate 64 gate rows and 64 up rows, or (mode 1,
// heads of 128) q | k | v with the per-head norms, the rotation and the write into the
// paged cache. In mode 1 a residual epilogue can also leave the input of the RMSNorm that
// follows (the new residual times the norm's weight, and its sums of squares), and every
// epilogue can scale its rows by the factor such a norm still owes (see TcParams): a
// decode step then runs no norm kernel between its products. A many-token variant walks
// its tiles with one block per SM (gemm_tc_persistent_kernel).
//
// Every block loads its own tiles (no multicast). Every wait on an mbarrier is bounded
// (llmrs_tc_set_wait_limit polls, 2^22 by default): when a wait runs out the block raises a flag
// in its shared memory, at which every other wait of the block returns too; the block then
// waits (bounded) for its copies and MMAs in flight, records a code in *error_flag, lets its
// epilogue write nothing (zeros into a cluster's sums), frees its tensor memory and returns.
//
// The reference's products are library calls (llm-core/src/backends/candle.rs:1276-1340).
#include <cuda.h>
#include <mutex>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

constexpr int TC_BM = 128;        // rows of A per tile = M of the MMA
constexpr int TC_BK = 64;         // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int TC_THREADS = 128;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;  // default polls of a barrier before giving up (a second or so)

enum TcEpilogue : int { TC_STORE = 0, TC_RESIDUAL = 1, TC_SILU_MUL = 2, TC_QKV_ROPE = 3 };

// What the epilogue TC_QKV_ROPE needs beside the product: the rows of W are the heads of q, then of k,
// then of v (128 features each); q gets its per-head norm and rotation and goes to q_out, k the same and
// goes to its page of the cache, v goes to its page as it is.
struct QkvRope {
  __nv_bfloat16* q_out;        // [tokens, ldq]
  long long ldq;
  __nv_bfloat16* cache;        // one layer's [n_pages, n_kv_heads, 2, page_size, 128]
  const float* q_norm_w;       // [128] or null
  const float* k_norm_w;
  const float* cos_sin;        // [positions, 64, 2] or null
  const int* positions;        // per token
  const int* token_req;        // per token: row of the block table
  const int* block_table;
  int table_stride, n_q_heads, n_kv_heads, page_size;
  float eps;
};

struct TcParams {
  void* out;            // TC_STORE / TC_SILU_MUL: [tokens, ldo] of out_dtype; TC_RESIDUAL: float32 h
  long long ldo;
  int out_dtype;        // LLMRS_F32 or LLMRS_BF16 (TC_STORE, TC_SILU_MUL)
  int epilogue;
  int a_rows, b_rows;   // valid extents (tokens / features according to the mode)
  int k_blocks;         // ceil(K / 64)
  int* error_flag;
  L2Prefetch next;      // mode 1: the start of the weights the next kernel streams, to be brought into the L2
  uint32_t wait_limit;  // polls of a barrier before a wait gives up
  int test_skip_kb;     // tests only: the producer leaves out the copy of its k block with this index (-1: none)
  QkvRope qr;           // TC_QKV_ROPE only
  // A norm that is spread over two products. The product BEFORE the norm (TC_RESIDUAL) also writes
  // emit_xw = (h + product) * emit_w in bfloat16, the norm's input times its weight, and leaves the sum of
  // squares of the features of h that a tile holds (128, or 256 with many tokens) in emit_part[tile][token]. The
  // product AFTER the norm takes emit_xw as its x and multiplies its rows by 1/sqrt(sum / scale_dim +
  // scale_eps), sum being the scale_parts entries of scale_part for the row's token, added in order.
  const float* emit_w;
  bf16* emit_xw;
  long long emit_ld;
  float* emit_part;
  const float* scale_part;
  int part_stride;      // tokens per row of emit_part / scale_part
  int scale_parts, scale_dim;
  float scale_eps;
};

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. False: gave up (or another thread of the block already had).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit, volatile int* abort_flag) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 128) {
      __nanosleep(64);
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}
// Bounded wait of a block that has given up already, for what it still has in flight (copies into its shared
// memory, MMAs into its tensor memory): the flag does not cut it short.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return;
    if (it > 128) __nanosleep(64);
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool tc_elect_one() {
  uint32_t leader;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(leader));
  return leader != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)1 << 16;                   // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t tc_instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// The barrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 consecutive float32 columns of this thread's lane.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// Four consecutive floats at `local_addr` (16-byte aligned) of the shared memory of block `rank` of the cluster.
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

// ---- the kernel ----------------------------------------------------------------------------
// MODE 0: rows of the tile are tokens (A = x), columns features (B = W); one block per tile.
// MODE 1: rows are features (A = W), columns tokens (B = x); gridDim.z = cluster size = k splits.
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcParams p) {
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ __align__(1024) unsigned char smem[];
  // Tiles need 1024-byte alignment for the 128-byte swizzle pattern.
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y;
  const int splits = MODE == 1 ? (int)gridDim.z : 1;
  const int split = MODE == 1 ? (int)blockIdx.z : 0;
  const int kb0 = (int)(((long long)split * p.k_blocks) / splits);
  const int kb1 = (int)(((long long)(split + 1) * p.k_blocks) / splits);
  const int nkb = kb1 - kb0;

  // Row scales of a product that follows a norm spread over two products (see TcParams).
  __shared__ float inv_s[64], inv_part[64];
  const bool scaled = MODE == 1 && p.scale_part != nullptr;

  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + STAGES), accum_bar = tc_smem(bars + 2 * STAGES);
  const int early = MODE == 1 ? min(nkb, STAGES) : 0;   // stages whose weight tile is requested before the wait
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Mode 1, the epilogue's work: the tokens of the tile are dealt out over the blocks of the cluster (block `rank`
  // owns tokens rank, rank + splits, ...), and an item is a token of the block and a quad q: features 4q..4q+3 and
  // 64+4q..64+4q+3 of the tile's 128, i.e. four of the pairs (i, i + 64) that SiLU*up and the rotation combine.
  // Thread etid takes items etid, etid + 128, ...: warps 2 and 3, which have nothing to do while the product runs,
  // own the first ones and fetch what those need from global memory (the residual's old values, the next norm's
  // weight, position, page, rotation) under the product instead of after it.
  const int etid = MODE == 1 ? ((tid + 64) & (TC_THREADS - 1)) : tid;
  const uint32_t rank = (MODE == 1 && splits > 1) ? cluster_rank() : 0u;
  const int n_tok = MODE == 1 ? min(BN, p.b_rows - tile_b * BN) : 0;
  const int n_mine = n_tok > (int)rank ? (n_tok - 1 - (int)rank) / splits + 1 : 0;   // tokens this block owns
  const int n_items = n_mine * 16;
  bool pf = false;
  float4 pf_a = make_float4(0.f, 0.f, 0.f, 0.f), pf_b = pf_a, pf_c = pf_a, pf_d = pf_a;   // residual: h lo/hi, w lo/hi; q|k|v: rotation
  int pf_pos = 0, pf_page = 0;

  int issued = 0;                      // thread 0: k blocks whose copies it has requested
  const int skip = p.test_skip_kb;     // -1 outside the test of the bounded waits
  if (warp == 0 && lane == 0) {
    // Producer: one thread feeds the ring of stages by TMA. In mode 1 the A operand is the
    // weight, which no earlier kernel writes: its first tiles are requested before the
    // wait on the preceding kernel, whose tail they overlap. (Requesting them still earlier, before
    // tensor memory is allocated, made the decode step slower: 3.83 -> 3.96 ms.)
    for (int i = 0; i < early; ++i) {
      if (i == skip) continue;
      mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
      tma_load_2d(tc_smem(tiles + (size_t)i * STAGE_BYTES), &map_a, full0 + 8 * i, (kb0 + i) * TC_BK, tile_a * TC_BM);
    }
    pdl_wait();
    for (int i = 0; i < early; ++i) {
      if (i == skip) continue;
      tma_load_2d(tc_smem(tiles + (size_t)i * STAGE_BYTES) + A_BYTES, &map_b, full0 + 8 * i, (kb0 + i) * TC_BK,
                  tile_b * BN);
    }
    issued = early;
    for (int i = early; i < nkb; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES && !mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, p.wait_limit, abort_flag)) break;
      issued = i + 1;
      if (i == skip) continue;
      mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
      const uint32_t a_dst = tc_smem(tiles + (size_t)s * STAGE_BYTES);
      tma_load_2d(a_dst, &map_a, full0 + 8 * s, (kb0 + i) * TC_BK, tile_a * TC_BM);
      tma_load_2d(a_dst + A_BYTES, &map_b, full0 + 8 * s, (kb0 + i) * TC_BK, tile_b * BN);
    }
  } else if (warp == 1) {
    // MMA issuer: four k16 steps per stage. The whole warp walks the loop and computes the operands, one
    // elected lane issues: operands that are the same in all lanes stay in uniform registers, where the
    // MMA wants them (issued from a one-thread branch each MMA costs its thread over a hundred cycles).
    constexpr uint32_t idesc = tc_instr_desc(BN);
    const bool leader = tc_elect_one();
    for (int i = 0; i < nkb; ++i) {
      const int s = i % STAGES;
      if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, (i / STAGES) & 1, p.wait_limit, abort_flag))) break;
      tc_fence_after();
      const uint32_t a_addr = tc_smem(tiles + (size_t)s * STAGE_BYTES);
      const uint64_t a_desc = tc_smem_desc(a_addr), b_desc = tc_smem_desc(a_addr + A_BYTES);
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k)
        if (leader) tc_mma(tmem_base, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
      if (leader) tc_commit(empty0 + 8 * s);  // frees the stage when these MMAs are done
      __syncwarp();
    }
    if (leader) tc_commit(accum_bar);
  } else if (MODE == 1 && warp >= 2) {
    pdl_wait();
    if (etid < n_items) {      // the thread's first item
      const int j = (int)rank + splits * (etid >> 4), q = etid & 15, t = tile_b * BN + j;
      if (p.epilogue == TC_RESIDUAL) {
        const int f_lo = tile_a * TC_BM + 4 * q, f_hi = f_lo + 64;
        const float* h = (const float*)p.out + (size_t)t * p.ldo;
        if (f_lo < p.a_rows) { pf_a = *reinterpret_cast<const float4*>(h + f_lo); if (p.emit_w) pf_c = *reinterpret_cast<const float4*>(p.emit_w + f_lo); }
        if (f_hi < p.a_rows) { pf_b = *reinterpret_cast<const float4*>(h + f_hi); if (p.emit_w) pf_d = *reinterpret_cast<const float4*>(p.emit_w + f_hi); }
        pf = true;
      } else if (p.epilogue == TC_QKV_ROPE) {
        const QkvRope& g = p.qr;
        pf_pos = g.positions[t];
        if (tile_a >= g.n_q_heads)
          pf_page = LLMRS_CHECKED_PAGE(g.block_table[(size_t)g.token_req[t] * g.table_stride + pf_pos / g.page_size], 5, t);
        if (g.cos_sin && tile_a < g.n_q_heads + g.n_kv_heads) {
          const float4* cs = reinterpret_cast<const float4*>(g.cos_sin + ((size_t)pf_pos * 64 + 4 * q) * 2);
          pf_a = cs[0];
          pf_b = cs[1];
        }
        pf = true;
      }
    }
    if (p.scale_part) {
      // While the product runs: the row scales 1/sqrt(sum of the pieces / dim + eps) of this
      // tile's tokens. A piece's row holds all tokens side by side, so the 64 threads read whole rows:
      // n_pow tokens wide, 64 / n_pow rows at a time; the groups' sums are then added in order.
      const int u = tid - 64;
      const int n_tok_s = min(BN, p.b_rows - tile_b * BN);
      int n_pow = 1;
      while (n_pow < n_tok_s) n_pow <<= 1;
      const int j = u % n_pow, g = u / n_pow, n_groups = 64 / n_pow;
      float ss = 0.f;
      if (j < n_tok_s) {
        const float* src = p.scale_part + tile_b * BN + j;
#pragma unroll 8
        for (int q = g; q < p.scale_parts; q += n_groups) ss += __ldcg(src + (size_t)q * p.part_stride);
      }
      inv_part[u] = ss;
      asm volatile("bar.sync 1, 64;" ::: "memory");
      if (u < n_tok_s) {
        float sum = 0.f;
        for (int k = 0; k < n_groups; ++k) sum += inv_part[k * n_pow + u];
        inv_s[u] = 1.0f / sqrtf(sum / (float)p.scale_dim + p.scale_eps);
      }
    }
  }
  __syncwarp();
  if (nkb > 0) mbar_wait(accum_bar, 0, p.wait_limit, abort_flag);
  tc_fence_after();
  // Every MMA has finished (accumulator barrier), so the stages are free for the epilogue's use; and from
  // here on all threads agree on whether the block gave up: tcgen05.ld below is warp-wide, and a cluster's
  // barriers want every block.
  __syncthreads();
  const bool ok = *abort_flag == 0;
  if (!ok) {
    // MMAs that were issued before the block gave up write tensor memory and read the stages: they are
    // waited for (their commit on the accumulator barrier was issued all the same) before either is touched.
    if (warp == 1 && nkb > 0) mbar_drain(accum_bar, 0, p.wait_limit);
    if (tid == 0) {
      // Nor may copies still land in this block's shared memory, which the epilogue reuses.
      for (int i = max(0, issued - STAGES); i < issued; ++i)
        if (i != skip) mbar_drain(full0 + 8 * (i % STAGES), (i / STAGES) & 1, p.wait_limit);
      if (p.error_flag) atomicExch(p.error_flag, 1);
    }
    tc_fence_after();
    __syncthreads();
  }

  pdl_wait();  // the epilogue writes (and for the residual reads) what earlier kernels touch
  const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int row = warp * 32 + lane;  // row of the tile this thread reads from tensor memory

  if (MODE == 0) {
    // Rows are tokens: each thread owns one token's BN features.
    const int t = tile_a * TC_BM + row;
    const bool t_ok = t < p.a_rows && ok;
    if (p.epilogue == TC_SILU_MUL) {
      // Columns come in groups of 128: 64 gate columns, then the 64 up columns of the same features.
#pragma unroll 1
      for (int g = 0; g < BN / 128; ++g) {
#pragma unroll 1
        for (int c = 0; c < 64; c += 8) {
          float gv[8], uv[8];
          tc_ld8(taddr + g * 128 + c, gv);
          tc_ld8(taddr + g * 128 + 64 + c, uv);
          const int f = (tile_b * BN + g * 128) / 2 + c;
          if (t_ok && f < p.b_rows / 2) {
            bf16* o = (bf16*)p.out + (size_t)t * p.ldo + f;
            uint4 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h2[e] = __floats2bfloat162_rn(silu_f(gv[2 * e]) * uv[2 * e], silu_f(gv[2 * e + 1]) * uv[2 * e + 1]);
            *reinterpret_cast<uint4*>(o) = pk;
          }
          __syncwarp();
        }
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 8) {
        float v[8];
        tc_ld8(taddr + c, v);
        const int f = tile_b * BN + c;
        if (!t_ok || f >= p.b_rows) {
          // nothing to store for this thread; stay with the warp for the next tcgen05.ld
        } else if (p.epilogue == TC_RESIDUAL) {
          float4* hp = reinterpret_cast<float4*>((float*)p.out + (size_t)t * p.ldo + f);
          float4 x0 = hp[0], x1 = hp[1];
          x0.x += v[0]; x0.y += v[1]; x0.z += v[2]; x0.w += v[3];
          x1.x += v[4]; x1.y += v[5]; x1.z += v[6]; x1.w += v[7];
          hp[0] = x0; hp[1] = x1;
        } else if (p.out_dtype == LLMRS_F32) {
          float4* op = reinterpret_cast<float4*>((float*)p.out + (size_t)t * p.ldo + f);
          op[0] = make_float4(v[0], v[1], v[2], v[3]);
          op[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          uint4 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
          *reinterpret_cast<uint4*>((bf16*)p.out + (size_t)t * p.ldo + f) = pk;
        }
        __syncwarp();
      }
    }
    tc_fence_before();
    __syncthreads();
  } else {
    // Rows are features, columns tokens. Partial tile -> shared memory, token-major -> every block sums, over the
    // cluster's blocks in rank order, the tokens it owns -> epilogue. A thread's item is 2 x 4 neighbouring features of
    // one token: 16-byte loads, through the cluster too, and all of an item's loads are issued before the first is used.
    // [BN tokens][RT]; the stages are free (see the join above).
    float* red = reinterpret_cast<float*>(tiles);
    // This block's stream is over; what is left is its epilogue: the memory system can serve the next kernel.
    if (tid == 0) l2_prefetch_slice(p.next);
    constexpr int RT = TC_BM + 4;     // a token's row: 16-byte aligned, and neighbouring tokens four banks apart
#pragma unroll 1
    for (int c = 0; c < BN; c += 8) {
      float v[8];
      if (nkb > 0 && ok) {
        tc_ld8(taddr + c, v);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) red[(c + e) * RT + row] = v[e];
    }
    tc_fence_before();
    if (splits > 1) cluster_sync_all(); else __syncthreads();

    const uint32_t red_addr = tc_smem(red);
    const QkvRope& g = p.qr;
    // q|k|v: the tile is one head.
    const int kind = tile_a < g.n_q_heads ? 0 : tile_a < g.n_q_heads + g.n_kv_heads ? 1 : 2;
    const int hidx = kind == 0 ? tile_a : kind == 1 ? tile_a - g.n_q_heads : tile_a - g.n_q_heads - g.n_kv_heads;
    for (int base = 0; base < n_items; base += TC_THREADS) {   // every thread walks the loop (warp shuffles below)
      const int it = base + etid;
      const bool live = it < n_items;
      const bool fetched = pf && base == 0;
      const int q = it & 15;
      const int j = (int)rank + splits * (live ? it >> 4 : 0);      // a thread without an item works on the block's first token, stores nothing
      const int t = tile_b * BN + j;
      const int f_lo = tile_a * TC_BM + 4 * q, f_hi = f_lo + 64;     // features come in eights: a quad is whole or absent
      const bool lo_ok = live && f_lo < p.a_rows, hi_ok = live && f_hi < p.a_rows;
      // What the item needs from global memory is asked for before the sums over the cluster, so that the
      // latencies overlap.
      float4 ga = pf_a, gb = pf_b, gc = pf_c, gd = pf_d;
      int pos = pf_pos, page = pf_page;
      if (!fetched) {
        if (p.epilogue == TC_RESIDUAL) {
          const float* h = (const float*)p.out + (size_t)t * p.ldo;
          if (lo_ok) { ga = *reinterpret_cast<const float4*>(h + f_lo); if (p.emit_w) gc = *reinterpret_cast<const float4*>(p.emit_w + f_lo); }
          if (hi_ok) { gb = *reinterpret_cast<const float4*>(h + f_hi); if (p.emit_w) gd = *reinterpret_cast<const float4*>(p.emit_w + f_hi); }
        } else if (p.epilogue == TC_QKV_ROPE && live) {
          pos = g.positions[t];
          if (kind != 0)
            page = LLMRS_CHECKED_PAGE(g.block_table[(size_t)g.token_req[t] * g.table_stride + pos / g.page_size], 5, t);
          if (g.cos_sin && kind != 2) {
            const float4* cs = reinterpret_cast<const float4*>(g.cos_sin + ((size_t)pos * 64 + 4 * q) * 2);
            ga = cs[0];
            gb = cs[1];
          }
        }
      }
      float lo[4], hi[4];
      {
        const uint32_t a_lo = red_addr + (uint32_t)(j * RT + 4 * q) * 4, a_hi = a_lo + 64 * 4;
        float4 sl, sh;
        if (splits > 1) {
          float4 vl[8], vh[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (r < splits) {
              vl[r] = ld_cluster_f32x4(a_lo, (uint32_t)r);
              vh[r] = ld_cluster_f32x4(a_hi, (uint32_t)r);
            }
          sl = vl[0];
          sh = vh[0];
#pragma unroll
          for (int r = 1; r < 8; ++r)
            if (r < splits) {       // in rank order
              sl.x += vl[r].x; sl.y += vl[r].y; sl.z += vl[r].z; sl.w += vl[r].w;
              sh.x += vh[r].x; sh.y += vh[r].y; sh.z += vh[r].z; sh.w += vh[r].w;
            }
        } else {
          sl = *reinterpret_cast<const float4*>(red + j * RT + 4 * q);
          sh = *reinterpret_cast<const float4*>(red + j * RT + 4 * q + 64);
        }
        const float sc = scaled ? inv_s[j] : 1.f;
        lo[0] = sl.x * sc; lo[1] = sl.y * sc; lo[2] = sl.z * sc; lo[3] = sl.w * sc;
        hi[0] = sh.x * sc; hi[1] = sh.y * sc; hi[2] = sh.z * sc; hi[3] = sh.w * sc;
      }
      if (p.epilogue == TC_SILU_MUL) {
        // The tile's first 64 rows are gate rows, the other 64 the up rows of the same features.
        const int f = tile_a * (TC_BM / 2) + 4 * q;
        if (live && f < p.a_rows / 2) {
          uint2 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
          h2[0] = __floats2bfloat162_rn(silu_f(lo[0]) * hi[0], silu_f(lo[1]) * hi[1]);
          h2[1] = __floats2bfloat162_rn(silu_f(lo[2]) * hi[2], silu_f(lo[3]) * hi[3]);
          *reinterpret_cast<uint2*>((bf16*)p.out + (size_t)t * p.ldo + f) = pk;
        }
      } else if (p.epilogue == TC_RESIDUAL) {
        float* h = (float*)p.out + (size_t)t * p.ldo;
        const float4 n_lo = make_float4(ga.x + lo[0], ga.y + lo[1], ga.z + lo[2], ga.w + lo[3]);
        const float4 n_hi = make_float4(gb.x + hi[0], gb.y + hi[1], gb.z + hi[2], gb.w + hi[3]);
        if (lo_ok) *reinterpret_cast<float4*>(h + f_lo) = n_lo;
        if (hi_ok) *reinterpret_cast<float4*>(h + f_hi) = n_hi;
        if (p.emit_w) {
          // The norm that follows: its input times its weight, and the sum of squares of the token's 128 features
          // of this tile (the 16 threads of a token sit side by side in a warp).
          float ss = 0.f;
          if (lo_ok) {
            uint2 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
            h2[0] = __floats2bfloat162_rn(n_lo.x * gc.x, n_lo.y * gc.y);
            h2[1] = __floats2bfloat162_rn(n_lo.z * gc.z, n_lo.w * gc.w);
            *reinterpret_cast<uint2*>(p.emit_xw + (size_t)t * p.emit_ld + f_lo) = pk;
            ss += n_lo.x * n_lo.x + n_lo.y * n_lo.y + n_lo.z * n_lo.z + n_lo.w * n_lo.w;
          }
          if (hi_ok) {
            uint2 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
            h2[0] = __floats2bfloat162_rn(n_hi.x * gd.x, n_hi.y * gd.y);
            h2[1] = __floats2bfloat162_rn(n_hi.z * gd.z, n_hi.w * gd.w);
            *reinterpret_cast<uint2*>(p.emit_xw + (size_t)t * p.emit_ld + f_hi) = pk;
            ss += n_hi.x * n_hi.x + n_hi.y * n_hi.y + n_hi.z * n_hi.z + n_hi.w * n_hi.w;
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (live && q == 0) p.emit_part[(size_t)tile_a * p.part_stride + t] = ss;
        }
      } else if (p.epilogue == TC_QKV_ROPE) {
        if (kind != 2) {
          const float* w = kind == 0 ? g.q_norm_w : g.k_norm_w;
          if (w) {
            float ss = lo[0] * lo[0] + lo[1] * lo[1] + lo[2] * lo[2] + lo[3] * lo[3] +
                       hi[0] * hi[0] + hi[1] * hi[1] + hi[2] * hi[2] + hi[3] * hi[3];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = 1.0f / sqrtf(ss / 128.0f + g.eps);
            const float4 w_lo = *reinterpret_cast<const float4*>(w + 4 * q), w_hi = *reinterpret_cast<const float4*>(w + 64 + 4 * q);
            lo[0] *= inv * w_lo.x; lo[1] *= inv * w_lo.y; lo[2] *= inv * w_lo.z; lo[3] *= inv * w_lo.w;
            hi[0] *= inv * w_hi.x; hi[1] *= inv * w_hi.y; hi[2] *= inv * w_hi.z; hi[3] *= inv * w_hi.w;
          }
          if (g.cos_sin) {
            // (cos, sin) of the pairs 4q..4q+3: feature i turns with feature i + 64.
            const float c[4] = {ga.x, ga.z, gb.x, gb.z}, sn[4] = {ga.y, ga.w, gb.y, gb.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float a0 = lo[e] * c[e] - hi[e] * sn[e], b0 = hi[e] * c[e] + lo[e] * sn[e];
              lo[e] = a0;
              hi[e] = b0;
            }
          }
        }
        if (live) {
          bf16* dst;
          if (kind == 0) {
            dst = g.q_out + (size_t)t * g.ldq + (size_t)hidx * 128;
          } else {
            dst = g.cache + kv_tile_offset(page, hidx, kind - 1, g.n_kv_heads, g.page_size, 128) +
                  (size_t)(pos % g.page_size) * 128;
          }
          uint2 pl, ph;
          __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&pl);
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&ph);
          l2[0] = __floats2bfloat162_rn(lo[0], lo[1]); l2[1] = __floats2bfloat162_rn(lo[2], lo[3]);
          h2[0] = __floats2bfloat162_rn(hi[0], hi[1]); h2[1] = __floats2bfloat162_rn(hi[2], hi[3]);
          *reinterpret_cast<uint2*>(dst + 4 * q) = pl;
          *reinterpret_cast<uint2*>(dst + 64 + 4 * q) = ph;
        }
      } else if (p.out_dtype == LLMRS_F32) {
        float* o = (float*)p.out + (size_t)t * p.ldo;
        if (lo_ok) *reinterpret_cast<float4*>(o + f_lo) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        if (hi_ok) *reinterpret_cast<float4*>(o + f_hi) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      } else {
        bf16* o = (bf16*)p.out + (size_t)t * p.ldo;
        uint2 pl, ph;
        __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&pl);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&ph);
        l2[0] = __floats2bfloat162_rn(lo[0], lo[1]); l2[1] = __floats2bfloat162_rn(lo[2], lo[3]);
        h2[0] = __floats2bfloat162_rn(hi[0], hi[1]); h2[1] = __floats2bfloat162_rn(hi[2], hi[3]);
        if (lo_ok) *reinterpret_cast<uint2*>(o + f_lo) = pl;
        if (hi_ok) *reinterpret_cast<uint2*>(o + f_hi) = ph;
      }
    }
    // No block may leave while another still reads its shared memory.
    if (splits > 1) cluster_sync_all(); else __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- the persistent kernel for many tokens ----------------------------------------------------
// Rows of a tile are tokens (A = x), columns features (B = W), tiles of 128 x 256. One block per SM
// walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (token tiles of one feature tile side by side, so
// the blocks that run together share weights in L2). Warp 0 copies (TMA), warp 1 issues the MMAs, warps
// 2-5 run the epilogue. The accumulator is double-buffered in tensor memory (2 x 256 columns): the
// epilogue of a tile runs under the MMAs of the next one, and the ring of stages never drains between
// tiles.
constexpr int PS_BN = 256, PS_STAGES = 4, PS_THREADS = 192;
constexpr uint32_t PS_A_BYTES = TC_BM * TC_BK * 2, PS_B_BYTES = PS_BN * TC_BK * 2, PS_STAGE_BYTES = PS_A_BYTES + PS_B_BYTES;

// The residual stream's old values for the epilogue warps of the many-token kernels. In tensor memory a lane owns a
// token's row, and rows of h lie kilobytes apart: loaded by the lanes themselves, a tile's 8,192 values per warp came
// in at the latency of 32 round trips to memory (30 us a tile, longer than the tile's MMAs). Instead TMA brings
// pieces of 32 rows x 32 columns (128-byte swizzle, so that a lane reads its row without bank conflicts) into two
// buffers per warp, two pieces ahead of their use and across tiles.
constexpr uint32_t HF_PIECE_BYTES = 32 * 32 * 4;
struct HFeed {
  uint32_t buf0 = 0;            // the warp's first buffer in shared memory (the second lies HF_PIECE_BYTES on)
  uint32_t bar0 = 0;            // its first barrier (the second 8 bytes on)
  long long issued = 0, taken = 0;   // pieces requested / used
};
__device__ __forceinline__ void hfeed_request(const CUtensorMap* map_h, HFeed& hf, int col, int row, bool leader_lane) {
  if (leader_lane) {
    const uint32_t b = (uint32_t)(hf.issued & 1);
    // The lanes' reads of the buffer (generic proxy) come before the copy into it (async proxy).
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_tx(hf.bar0 + 8 * b, HF_PIECE_BYTES);
    tma_load_2d(hf.buf0 + HF_PIECE_BYTES * b, map_h, hf.bar0 + 8 * b, col, row);
  }
  ++hf.issued;
}
// The first two pieces of a tile (before its loop; later pieces are requested as earlier ones are used).
__device__ __forceinline__ void hfeed_start(const CUtensorMap* map_h, HFeed& hf, int tn, int tok0, bool leader_lane) {
  hfeed_request(map_h, hf, tn * 256, tok0, leader_lane);
  hfeed_request(map_h, hf, tn * 256 + 32, tok0, leader_lane);
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// The factor a norm spread over two products still owes this token's row (see TcParams), 1 without one.
__device__ __forceinline__ float ps_row_scale(const TcParams& p, int tok, bool t_ok) {
  if (!p.scale_part || !t_ok) return 1.f;
  float ss = 0.f;
  for (int q = 0; q < p.scale_parts; ++q) ss += __ldcg(p.scale_part + (size_t)q * p.part_stride + tok);
  return 1.0f / sqrtf(ss / (float)p.scale_dim + p.scale_eps);
}

// The epilogue of one tile of 256 columns whose rows are tokens, for one warp: `taddr` its 32 lanes of tensor memory
// at the tile's first column, `tok0` the token of lane 0 (lane l owns token tok0 + l), `tn` the tile's index along the
// features. TC_RESIDUAL: `hf` feeds the old values of h; the first two pieces of this tile have been requested, and
// those of the warp's next tile (next_tn, next_tok0; next_tn < 0: none) are requested here. All 32 lanes walk it
// together (tcgen05.ld is warp-wide) whether their token exists or not. False: a wait ran out.
__device__ __forceinline__ bool ps_epilogue_tile(const TcParams& p, const CUtensorMap* map_h, HFeed& hf, uint32_t taddr,
                                                 int tok0, int lane, int tn, int next_tn, int next_tok0,
                                                 bool leader_lane, volatile int* abort_flag) {
  const int tok = tok0 + lane;
  const bool t_ok = tok < p.a_rows;
  const float inv = ps_row_scale(p, tok, t_ok);
  if (p.epilogue == TC_SILU_MUL) {
    // Columns come in groups of 128: 64 gate columns, then the 64 up columns of the same features.
#pragma unroll 1
    for (int g = 0; g < PS_BN / 128; ++g) {
#pragma unroll 1
      for (int c = 0; c < 64; c += 8) {
        float gv[8], uv[8];
        tc_ld8(taddr + g * 128 + c, gv);
        tc_ld8(taddr + g * 128 + 64 + c, uv);
        const int f = (tn * PS_BN + g * 128) / 2 + c;
        if (t_ok && f < p.b_rows / 2) {
          uint4 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            h2[e] = __floats2bfloat162_rn(silu_f(gv[2 * e] * inv) * (uv[2 * e] * inv),
                                          silu_f(gv[2 * e + 1] * inv) * (uv[2 * e + 1] * inv));
          *reinterpret_cast<uint4*>((bf16*)p.out + (size_t)tok * p.ldo + f) = pk;
        }
        __syncwarp();
      }
    }
  } else if (p.epilogue == TC_RESIDUAL) {
    // h += y, 32 columns at a time. With emit_w the same pass writes the input of the norm that follows,
    // (h + y) * w in bfloat16, and adds up the squares of the lane's row.
    float* hrow = (float*)p.out + (size_t)tok * p.ldo;
    float ss = 0.f;
#pragma unroll 1
    for (int c = 0; c < PS_BN; c += 32) {
      float v[32];
      tc_ld32(taddr + c, v);
      const uint32_t b = (uint32_t)(hf.taken & 1);
      if (!__all_sync(0xffffffffu, mbar_wait(hf.bar0 + 8 * b, (uint32_t)(hf.taken >> 1) & 1, p.wait_limit, abort_flag)))
        return false;
      const uint32_t row_addr = hf.buf0 + HF_PIECE_BYTES * b + (uint32_t)lane * 128;
      float4 hv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = ld_shared_f4(row_addr + (uint32_t)((j ^ (lane & 7)) << 4));
      ++hf.taken;
      __syncwarp();   // every lane has read the buffer: the piece after next may land in it
      if (c + 64 < PS_BN) hfeed_request(map_h, hf, tn * PS_BN + c + 64, tok0, leader_lane);
      else if (next_tn >= 0) hfeed_request(map_h, hf, next_tn * PS_BN + c + 64 - PS_BN, next_tok0, leader_lane);
      const int f = tn * PS_BN + c;
      if (t_ok) {
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          if (f + 4 * j >= p.b_rows) break;     // features come in eights
          float n[8];
          n[0] = hv[j].x + v[4 * j] * inv; n[1] = hv[j].y + v[4 * j + 1] * inv;
          n[2] = hv[j].z + v[4 * j + 2] * inv; n[3] = hv[j].w + v[4 * j + 3] * inv;
          n[4] = hv[j + 1].x + v[4 * j + 4] * inv; n[5] = hv[j + 1].y + v[4 * j + 5] * inv;
          n[6] = hv[j + 1].z + v[4 * j + 6] * inv; n[7] = hv[j + 1].w + v[4 * j + 7] * inv;
          float4* dst = reinterpret_cast<float4*>(hrow + f + 4 * j);
          dst[0] = make_float4(n[0], n[1], n[2], n[3]);
          dst[1] = make_float4(n[4], n[5], n[6], n[7]);
          if (p.emit_w) {
            const float4 w0 = *reinterpret_cast<const float4*>(p.emit_w + f + 4 * j);
            const float4 w1 = *reinterpret_cast<const float4*>(p.emit_w + f + 4 * j + 4);
            uint4 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
            h2[0] = __floats2bfloat162_rn(n[0] * w0.x, n[1] * w0.y);
            h2[1] = __floats2bfloat162_rn(n[2] * w0.z, n[3] * w0.w);
            h2[2] = __floats2bfloat162_rn(n[4] * w1.x, n[5] * w1.y);
            h2[3] = __floats2bfloat162_rn(n[6] * w1.z, n[7] * w1.w);
            *reinterpret_cast<uint4*>(p.emit_xw + (size_t)tok * p.emit_ld + f + 4 * j) = pk;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += n[e] * n[e];
          }
        }
      }
      __syncwarp();
    }
    if (p.emit_w && t_ok) p.emit_part[(size_t)tn * p.part_stride + tok] = ss;
  } else {
#pragma unroll 1
    for (int c = 0; c < PS_BN; c += 8) {
      float v[8];
      tc_ld8(taddr + c, v);
      const int f = tn * PS_BN + c;
      if (!t_ok || f >= p.b_rows) {
        // nothing to store for this thread; stay with the warp for the next tcgen05.ld
      } else if (p.out_dtype == LLMRS_F32) {
        float4* op = reinterpret_cast<float4*>((float*)p.out + (size_t)tok * p.ldo + f);
        op[0] = make_float4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        op[1] = make_float4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
      } else {
        uint4 pk;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e] * inv, v[2 * e + 1] * inv);
        *reinterpret_cast<uint4*>((bf16*)p.out + (size_t)tok * p.ldo + f) = pk;
      }
      __syncwarp();
    }
  }
  return true;
}

__global__ void __launch_bounds__(PS_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_h, const TcParams p, int n_m, int n_tiles) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  unsigned char* h_pieces = tiles + (size_t)PS_STAGES * PS_STAGE_BYTES;   // two pieces of h per epilogue warp (HFeed)
  // full[4], empty[4], acc_full[2], acc_empty[2], drain, then the epilogue warps' two barriers each
  uint64_t* bars = reinterpret_cast<uint64_t*>(h_pieces + 8 * HF_PIECE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PS_STAGES + 5 + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + PS_STAGES), acc_full0 = tc_smem(bars + 2 * PS_STAGES),
                 acc_empty0 = acc_full0 + 16, drain_bar = acc_full0 + 32;
  if (tid == 0) {
    for (int s = 0; s < 2 * PS_STAGES + 2; ++s) mbar_init(full0 + 8 * s, 1);
    mbar_init(acc_empty0, 128);
    mbar_init(acc_empty0 + 8, 128);
    mbar_init(drain_bar, 1);
    for (int s = 0; s < 8; ++s) mbar_init(drain_bar + 8 + 8 * s, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // x is what an earlier kernel wrote; the epilogue writes what earlier kernels read
  const int nkb = p.k_blocks;
  long long copies = 0;   // warp 0: stages whose copies it has requested
  HFeed hf;               // epilogue warps: their pieces of the residual stream

  if (warp == 0) {
    // Copies: the whole warp walks the loop, one elected lane issues.
    const bool leader = tc_elect_one();
    long long it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const int tm = t % n_m, tn = t / n_m;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = (int)(it % PS_STAGES);
        if (it >= PS_STAGES) {
          ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, (uint32_t)((it / PS_STAGES) - 1) & 1, p.wait_limit, abort_flag));
          if (!ok) break;
        }
        if (leader && it != p.test_skip_kb) {
          mbar_expect_tx(full0 + 8 * s, PS_STAGE_BYTES);
          const uint32_t a_dst = tc_smem(tiles + (size_t)s * PS_STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * TC_BK, tm * TC_BM);
          tma_load_2d(a_dst + PS_A_BYTES, &map_b, full0 + 8 * s, kb * TC_BK, tn * PS_BN);
        }
        __syncwarp();
      }
    }
    copies = it;
  } else if (warp == 1) {
    // MMAs: operands computed by the whole warp (they stay in uniform registers), issued by one elected lane.
    constexpr uint32_t idesc = tc_instr_desc(PS_BN);
    const bool leader = tc_elect_one();
    long long it = 0;
    int lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
      const int buf = lt & 1;
      if (lt >= 2) {   // the epilogue has read the tile before last out of this buffer
        ok = __all_sync(0xffffffffu, mbar_wait(acc_empty0 + 8 * buf, (uint32_t)((lt >> 1) - 1) & 1, p.wait_limit, abort_flag));
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t d_addr = tmem_base + (uint32_t)buf * PS_BN;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = (int)(it % PS_STAGES);
        ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, (uint32_t)(it / PS_STAGES) & 1, p.wait_limit, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = tc_smem(tiles + (size_t)s * PS_STAGE_BYTES);
        const uint64_t a_desc = tc_smem_desc(a_addr), b_desc = tc_smem_desc(a_addr + PS_A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)
          if (leader) tc_mma(d_addr, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        if (leader) tc_commit(empty0 + 8 * s);
        __syncwarp();
      }
      if (leader && ok) tc_commit(acc_full0 + 8 * buf);
      __syncwarp();
    }
  } else {
    // Epilogue: thread = one token row of the tile; a warp reaches the 32 lanes of tensor memory
    // that its index modulo 4 names.
    const int quarter = warp & 3;
    const bool leader = tc_elect_one();
    hf.buf0 = tc_smem(h_pieces) + (uint32_t)(warp - 2) * 2 * HF_PIECE_BYTES;
    hf.bar0 = drain_bar + 8 + (uint32_t)(warp - 2) * 16;
    if (p.epilogue == TC_RESIDUAL && (int)blockIdx.x < n_tiles)
      hfeed_start(&map_h, hf, blockIdx.x / n_m, (blockIdx.x % n_m) * TC_BM + quarter * 32, leader);
    int lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++lt) {
      const int tm = t % n_m, tn = t / n_m, buf = lt & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(acc_full0 + 8 * buf, (uint32_t)(lt >> 1) & 1, p.wait_limit, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * PS_BN;
      const int t_next = t + (int)gridDim.x;
      const bool more = t_next < n_tiles && p.epilogue == TC_RESIDUAL;
      ok = ps_epilogue_tile(p, &map_h, hf, taddr, tm * TC_BM + quarter * 32, lane, tn, more ? t_next / n_m : -1,
                            more ? (t_next % n_m) * TC_BM + quarter * 32 : 0, leader, abort_flag);
      if (!ok) break;
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // The block gave up. Before tensor memory is freed and the block leaves: the MMAs that were issued must be
    // done, and no copy may still be on its way into this block's shared memory.
    if (warp == 1) {
      if (tc_elect_one()) tc_commit(drain_bar);
      __syncwarp();
      mbar_drain(drain_bar, 0, p.wait_limit);
    } else if (tid == 0) {
      for (long long i = copies > PS_STAGES ? copies - PS_STAGES : 0; i < copies; ++i)
        if (i != p.test_skip_kb) mbar_drain(full0 + 8 * (int)(i % PS_STAGES), (uint32_t)(i / PS_STAGES) & 1, p.wait_limit);
      if (p.error_flag) atomicExch(p.error_flag, 1);
    } else if (warp >= 2) {
      for (long long i = hf.taken; i < hf.issued; ++i) mbar_drain(hf.bar0 + 8 * (uint32_t)(i & 1), (uint32_t)(i >> 1) & 1, p.wait_limit);
    }
    __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- the persistent kernel for many tokens on pairs of SMs (cta_group::2) ------------------------
// A thread-block cluster of two blocks owns a tile of 256 tokens x 256 features. Each block copies its 128 token
// rows of x and ITS HALF (128 feature rows) of the weight tile; one thread of the pair's first block (the leader)
// issues tcgen05.mma.cta_group::2, M = 256, N = 256, which reads A from each block's own shared memory and B from
// both, and leaves each block's 128 rows of the result in that block's tensor memory. Against the one-block
// kernel an SM reads half the B operand from its shared memory per flop and holds 32 KB instead of 48 KB a
// stage. The roles of a block: warp 0 copies (TMA), warp 1 issues the MMAs (leader only), warps 2-5 run the
// epilogue of the block's own rows. Barriers:
//   full[s]      (leader's) both blocks' copies of a stage have landed: each block's TMA completes its bytes on
//                the leader's barrier (cp.async.bulk.tensor ... .cta_group::2 allows a barrier in the peer block)
//   empty[s]     (each block's own) the MMAs that read the stage are done: tcgen05.commit, multicast to both blocks
//   acc_full[b]  (each block's own) the tile in accumulator buffer b is complete: tcgen05.commit, multicast
//   acc_empty[b] (leader's) both blocks' epilogues have read buffer b: one arrival per epilogue warp
// Every wait is bounded as in the other kernels; a block that gave up still meets its peer at the cluster barrier
// before tensor memory is freed.
constexpr int PR_STAGES = 6, PR_THREADS = 192;
constexpr uint32_t PR_HALF_BYTES = TC_BM * TC_BK * 2, PR_STAGE_BYTES = 2 * PR_HALF_BYTES;   // A rows + half of B

__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// A copy into this block's shared memory whose bytes are counted by a barrier that may lie in the pair's other block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// One arrival, in both blocks of the pair, on the barrier at this offset of shared memory, when every MMA issued
// so far by this thread has finished.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both) : "memory");
}
// The same on this block's barrier alone.
__device__ __forceinline__ void tc_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Bounded wait on a barrier that threads of the other block arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint32_t limit, volatile int* abort_flag) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (it > 128) {
      __nanosleep(64);
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}
// Instruction descriptor of the pair's MMA: bf16 x bf16 -> f32, both K-major, M = 256 over the two blocks, N = n.
__host__ __device__ constexpr uint32_t tc_instr_desc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// ACC_BUFS accumulator buffers of 256 columns: 2 (all 512 columns; the epilogue of a tile runs under the MMAs of the
// next) or 1.
template <int ACC_BUFS>
__global__ void __launch_bounds__(PR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_h, const TcParams p, int n_m, int n_tiles, int* tmem_seen) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  unsigned char* h_pieces = tiles + (size_t)PR_STAGES * PR_STAGE_BYTES;   // two pieces of h per epilogue warp (HFeed)
  // full[S], empty[S], acc_full[2], acc_empty[2], drain, then the epilogue warps' two barriers each
  uint64_t* bars = reinterpret_cast<uint64_t*>(h_pieces + 8 * HF_PIECE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PR_STAGES + 5 + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_rank();        // 0: the leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + PR_STAGES), acc_full0 = tc_smem(bars + 2 * PR_STAGES),
                 acc_empty0 = acc_full0 + 16, drain_bar = acc_full0 + 32;
  constexpr uint32_t COLS = ACC_BUFS * PS_BN;
  if (tid == 0) {
    for (int s = 0; s < 2 * PR_STAGES + 2; ++s) mbar_init(full0 + 8 * s, 1);
    mbar_init(acc_empty0, 8);        // one arrival from each of the four epilogue warps of both blocks
    mbar_init(acc_empty0 + 8, 8);
    mbar_init(drain_bar, 1);
    for (int s = 0; s < 8; ++s) mbar_init(drain_bar + 8 + 8 * s, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    // Both blocks of the pair allocate (the same columns in each block's tensor memory).
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "r"(COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tmem_seen && tid == 0) tmem_seen[blockIdx.x] = (int)tmem_base;   // tests: what each block was given
  pdl_wait();   // x is what an earlier kernel wrote; the epilogue writes what earlier kernels read
  const int nkb = p.k_blocks;
  long long copies = 0;   // warp 0: stages whose copies it has requested
  HFeed hf;               // epilogue warps: their pieces of the residual stream

  if (warp == 0) {
    // Copies: the whole warp walks the loop, one elected lane issues. The leader announces the bytes of both blocks.
    const bool leader_lane = tc_elect_one();
    long long it = 0;
    bool ok = true;
    for (int t = pair; t < n_tiles && ok; t += n_pairs) {
      const int tm = t % n_m, tn = t / n_m;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = (int)(it % PR_STAGES);
        if (it >= PR_STAGES) {
          ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, (uint32_t)((it / PR_STAGES) - 1) & 1, p.wait_limit, abort_flag));
          if (!ok) break;
        }
        if (leader_lane && it != p.test_skip_kb) {
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * PR_STAGE_BYTES);
          const uint32_t dst = tc_smem(tiles + (size_t)s * PR_STAGE_BYTES);
          const uint32_t bar = map_to_rank(full0 + 8 * s, 0u);
          tma_load_2d_pair(dst, &map_a, bar, kb * TC_BK, tm * 2 * TC_BM + (int)rank * TC_BM);
          tma_load_2d_pair(dst + PR_HALF_BYTES, &map_b, bar, kb * TC_BK, tn * PS_BN + (int)rank * (PS_BN / 2));
        }
        __syncwarp();
      }
    }
    copies = it;
  } else if (warp == 1) {
    if (rank == 0) {
      // MMAs of the pair: operands computed by the whole warp, issued by one elected lane of the leader.
      constexpr uint32_t idesc = tc_instr_desc_pair(PS_BN);
      const bool leader_lane = tc_elect_one();
      long long it = 0;
      int lt = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs, ++lt) {
        const int buf = lt % ACC_BUFS;
        if (lt >= ACC_BUFS) {   // both epilogues have read the tile that lay in this buffer
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(acc_empty0 + 8 * buf, (uint32_t)((lt / ACC_BUFS) - 1) & 1, p.wait_limit, abort_flag));
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t d_addr = tmem_base + (uint32_t)buf * PS_BN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = (int)(it % PR_STAGES);
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(full0 + 8 * s, (uint32_t)(it / PR_STAGES) & 1, p.wait_limit, abort_flag));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = tc_smem(tiles + (size_t)s * PR_STAGE_BYTES);
          const uint64_t a_desc = tc_smem_desc(a_addr), b_desc = tc_smem_desc(a_addr + PR_HALF_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            if (leader_lane) tc_mma_pair(d_addr, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          if (leader_lane) tc_commit_pair(empty0 + 8 * s);
          __syncwarp();
        }
        if (leader_lane && ok) tc_commit_pair(acc_full0 + 8 * buf);
        __syncwarp();
      }
    }
  } else {
    // Epilogue of this block's 128 token rows: thread = one row; a warp reaches the 32 lanes of tensor memory
    // that its index modulo 4 names.
    const int quarter = warp & 3;
    const bool leader_lane = tc_elect_one();
    const int row0 = (int)rank * TC_BM + quarter * 32;   // the warp's first row of a tile
    hf.buf0 = tc_smem(h_pieces) + (uint32_t)(warp - 2) * 2 * HF_PIECE_BYTES;
    hf.bar0 = drain_bar + 8 + (uint32_t)(warp - 2) * 16;
    if (p.epilogue == TC_RESIDUAL && pair < n_tiles)
      hfeed_start(&map_h, hf, pair / n_m, (pair % n_m) * 2 * TC_BM + row0, leader_lane);
    int lt = 0;
    bool ok = true;
    for (int t = pair; t < n_tiles && ok; t += n_pairs, ++lt) {
      const int tm = t % n_m, tn = t / n_m, buf = lt % ACC_BUFS;
      ok = __all_sync(0xffffffffu, mbar_wait(acc_full0 + 8 * buf, (uint32_t)(lt / ACC_BUFS) & 1, p.wait_limit, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * PS_BN;
      const int t_next = t + n_pairs;
      const bool more = t_next < n_tiles && p.epilogue == TC_RESIDUAL;
      ok = ps_epilogue_tile(p, &map_h, hf, taddr, tm * 2 * TC_BM + row0, lane, tn, more ? t_next / n_m : -1,
                            more ? (t_next % n_m) * 2 * TC_BM + row0 : 0, leader_lane, abort_flag);
      if (!ok) break;
      tc_fence_before();
      __syncwarp();   // the warp has read its lanes of the buffer
      if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty0 + 8 * buf, 0u));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // The block gave up. The MMAs that were issued must be done before tensor memory is freed, and the copies that
    // were requested must have landed (the leader's barriers count both blocks' bytes; the peer stays until the
    // cluster barrier below).
    if (rank == 0 && warp == 1) {
      if (tc_elect_one()) tc_commit_pair_local(drain_bar);
      __syncwarp();
      mbar_drain(drain_bar, 0, p.wait_limit);
    } else if (rank == 0 && tid == 0) {
      for (long long i = copies > PR_STAGES ? copies - PR_STAGES : 0; i < copies; ++i)
        if (i != p.test_skip_kb) mbar_drain(full0 + 8 * (int)(i % PR_STAGES), (uint32_t)(i / PR_STAGES) & 1, p.wait_limit);
    } else if (warp >= 2) {
      for (long long i = hf.taken; i < hf.issued; ++i) mbar_drain(hf.bar0 + 8 * (uint32_t)(i & 1), (uint32_t)(i >> 1) & 1, p.wait_limit);
    }
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    __syncthreads();
  }
  // Neither block may free tensor memory or leave while the other still computes into it or signals its barriers.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(COLS) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------------
static uint32_t g_tc_wait_limit = TC_WAIT_LIMIT;
static int g_tc_test_skip_kb = -1;

// Polls of a barrier before a wait of the tcgen05 product kernels gives up (0: the default, 2^22).
LLMRS_API void llmrs_tc_set_wait_limit(unsigned polls) { g_tc_wait_limit = polls ? polls : TC_WAIT_LIMIT; }

// For the test of the bounded waits only: the producers of the next launches leave out the copy of their
// k block with this index, so that a wait of every block runs out (-1, the default: every copy is made).
LLMRS_API void llmrs_tc_test_skip_copy(int k_block) { g_tc_test_skip_kb = k_block; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// Tensor map of a K-major bfloat16 matrix [rows, K] with row stride ld (elements); box = 64 x box_rows.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return llmrs_fail("gemm_bf16: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return llmrs_fail("gemm_bf16: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// Tensor map of the float32 residual stream [rows, cols] with row stride ld (elements) for the pieces of 32 x 32 that
// the many-token kernels' epilogue warps fetch (see HFeed).
static int make_map_h(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return llmrs_fail("gemm_bf16: cuTensorMapEncodeTiled is not available from this driver");
  LLMRS_REQUIRE(((uintptr_t)base & 15) == 0 && ld % 4 == 0, "gemm_bf16: the residual stream must be 16-byte aligned, rows too");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return llmrs_fail("gemm_bf16: cuTensorMapEncodeTiled (residual stream) failed with code %d", (int)r);
  return 0;
}

template <int BN, int STAGES, int MODE>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, int cluster_z,
                     cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("gemm_bf16: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster_z;
  cfg.numAttrs = 1;
  if (g_llmrs_pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, MODE>, ma, mb, p);
  if (e != cudaSuccess) return llmrs_fail("gemm_bf16 launch: %s", cudaGetErrorString(e));
  return llmrs_launch_status("gemm_bf16");
}

// The two halves of a norm that is spread over two products (see TcParams).
struct NormLink {
  const float* emit_w = nullptr;
  void* emit_xw = nullptr;
  long long emit_ld = 0;
  float* emit_part = nullptr;
  const float* scale_part = nullptr;
  int part_stride = 0, scale_parts = 0, scale_dim = 0;
  float scale_eps = 0.f;
};

static int gemm_bf16_impl(const void* x, long long ldx, const void* w, void* out, long long ldo, int tokens,
                          int features, int K, int epilogue, int out_dtype, int splits, int* error_flag,
                          const QkvRope* qr, const NormLink* nl, cudaStream_t stream);

// q | k | v = x Wqkv^T with the per-head norms, the rotation and the cache write in the product's
// epilogue (few tokens, heads of 128 features): q goes to q_out (bfloat16 [tokens, ldq]), k and v to the
// pages that block_table names for the tokens' positions. Same arithmetic as the product followed by
// llmrs_qk_norm_rope_kvwrite, without rounding q, k and v to bfloat16 in between.
LLMRS_API int llmrs_gemm_qkv_rope(const void* x, long long ldx, const void* w, int tokens, int K, int splits,
                                  void* q_out, long long ldq, void* cache, const float* q_norm_w,
                                  const float* k_norm_w, const float* cos_sin, const int* positions,
                                  const int* token_req, const int* block_table, int table_stride, int n_q_heads,
                                  int n_kv_heads, int page_size, float eps, const float* scale_part, int part_stride,
                                  int scale_parts, int scale_dim, float scale_eps, int* error_flag,
                                  cudaStream_t stream) {
  LLMRS_REQUIRE(tokens > 0 && tokens <= 64, "gemm_qkv_rope: takes 1 to 64 tokens, got %d", tokens);
  LLMRS_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && page_size > 0 && table_stride > 0, "gemm_qkv_rope: bad sizes");
  LLMRS_REQUIRE(q_out && cache && positions && token_req && block_table, "gemm_qkv_rope: missing argument");
  LLMRS_REQUIRE(((uintptr_t)q_out & 15) == 0 && ldq % 8 == 0 && ((uintptr_t)cache & 15) == 0 && ((uintptr_t)cos_sin & 15) == 0 &&
                    ((uintptr_t)q_norm_w & 15) == 0 && ((uintptr_t)k_norm_w & 15) == 0,
                "gemm_qkv_rope: q_out, the cache, the rotation table and the norm weights must be 16-byte aligned");
  QkvRope qr;
  qr.q_out = (__nv_bfloat16*)q_out; qr.ldq = ldq; qr.cache = (__nv_bfloat16*)cache; qr.q_norm_w = q_norm_w;
  qr.k_norm_w = k_norm_w; qr.cos_sin = cos_sin; qr.positions = positions; qr.token_req = token_req;
  qr.block_table = block_table; qr.table_stride = table_stride; qr.n_q_heads = n_q_heads; qr.n_kv_heads = n_kv_heads;
  qr.page_size = page_size; qr.eps = eps;
  NormLink nl;
  nl.scale_part = scale_part; nl.part_stride = part_stride; nl.scale_parts = scale_parts; nl.scale_dim = scale_dim;
  nl.scale_eps = scale_eps;
  return gemm_bf16_impl(x, ldx, w, q_out, ldq, tokens, (n_q_heads + 2 * n_kv_heads) * 128, K, TC_QKV_ROPE, LLMRS_BF16,
                        splits, error_flag, &qr, &nl, stream);
}

static int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mh, const TcParams& p,
                             int n_m, int n_tiles, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)PS_STAGES * PS_STAGE_BYTES + 8 * HF_PIECE_BYTES + (2 * PS_STAGES + 5 + 8) * 8 + 16;
  static int n_sm = 0;
  if (n_sm == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("gemm_bf16: shared memory %zu: %s", smem, cudaGetErrorString(e));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (n_sm <= 0) n_sm = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles < n_sm ? n_tiles : n_sm);
  cfg.blockDim = dim3(PS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cfg.numAttrs = 0;
  if (g_llmrs_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  cfg.attrs = attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_persistent_kernel, ma, mb, mh, p, n_m, n_tiles);
  if (e != cudaSuccess) return llmrs_fail("gemm_bf16 launch: %s", cudaGetErrorString(e));
  return llmrs_launch_status("gemm_bf16");
}

// Many tokens on pairs of SMs (gemm_tc_pair_kernel): as many clusters of two blocks as the device holds at a time.
static int g_tc_pairs = 1;

// 0: steps of many tokens stay on the one-block kernel (1, the default: the kernel on pairs of SMs from 129 tokens).
LLMRS_API void llmrs_tc_use_pairs(int on) { g_tc_pairs = on ? 1 : 0; }

template <int ACC_BUFS>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mh, const TcParams& p, int n_m,
                       int n_tiles, int* tmem_seen, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)PR_STAGES * PR_STAGE_BYTES + 8 * HF_PIECE_BYTES + (2 * PR_STAGES + 5 + 8) * 8 + 16;
  static int max_pairs = 0;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (max_pairs == 0) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<ACC_BUFS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return llmrs_fail("gemm_bf16: shared memory %zu: %s", smem, cudaGetErrorString(e));
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2);
      q.blockDim = dim3(PR_THREADS);
      q.dynamicSmemBytes = smem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<ACC_BUFS>, &q);
      if (e != cudaSuccess || n <= 0) return llmrs_fail("gemm_bf16: no room for a pair of blocks: %s", cudaGetErrorString(e));
      max_pairs = n;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (n_tiles < max_pairs ? n_tiles : max_pairs));
  cfg.blockDim = dim3(PR_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (g_llmrs_pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<ACC_BUFS>, ma, mb, mh, p, n_m, n_tiles, tmem_seen);
  if (e != cudaSuccess) return llmrs_fail("gemm_bf16 launch (pairs): %s", cudaGetErrorString(e));
  return llmrs_launch_status("gemm_bf16");
}

// The kernel on pairs of SMs by itself, for tests and measurements: acc_buffers accumulator tiles in tensor memory
// (1 or 2); tmem_seen (or null) receives, per block, the tensor-memory address the block was given.
LLMRS_API int llmrs_gemm_bf16_pairs(const void* x, long long ldx, const void* w, void* out, long long ldo, int tokens,
                                    int features, int K, int epilogue, int out_dtype, int acc_buffers, int* tmem_seen,
                                    int* error_flag, cudaStream_t stream) {
  LLMRS_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_bf16_pairs: unknown epilogue %d", epilogue);
  LLMRS_REQUIRE(acc_buffers == 1 || acc_buffers == 2, "gemm_bf16_pairs: 1 or 2 accumulator buffers");
  LLMRS_REQUIRE(tokens > 0 && features > 0 && K > 0, "gemm_bf16_pairs: bad sizes");
  LLMRS_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && features % 8 == 0 && ldo % 8 == 0,
                "gemm_bf16_pairs: K, features and the row strides must be multiples of 8");
  LLMRS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16_pairs: operands must be 16-byte aligned");
  LLMRS_REQUIRE(epilogue != TC_SILU_MUL || features % 256 == 0,
                "gemm_bf16_pairs: SiLU*up needs features in groups of 256, got %d", features);
  TcParams p = {};
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.k_blocks = (K + TC_BK - 1) / TC_BK; p.error_flag = error_flag;
  p.wait_limit = g_tc_wait_limit; p.test_skip_kb = g_tc_test_skip_kb;
  p.a_rows = tokens; p.b_rows = features;
  CUtensorMap ma, mb, mh = {};
  int rc;
  if ((rc = make_map(&ma, x, tokens, K, ldx, TC_BM))) return rc;
  if ((rc = make_map(&mb, w, features, K, K, PS_BN / 2))) return rc;
  if (epilogue == TC_RESIDUAL && (rc = make_map_h(&mh, out, tokens, features, ldo))) return rc;
  const int n_m = (tokens + 2 * TC_BM - 1) / (2 * TC_BM), n_n = (features + PS_BN - 1) / PS_BN;
  if (acc_buffers == 1) return launch_pair<1>(ma, mb, mh, p, n_m, n_m * n_n, tmem_seen, stream);
  return launch_pair<2>(ma, mb, mh, p, n_m, n_m * n_n, tmem_seen, stream);
}

// y = x W^T for bfloat16 x [tokens, K] (row stride ldx) and W [features, K] (dense).
//   epilogue TC_STORE:    out[tokens, features] (out_dtype), row stride ldo
//   epilogue TC_RESIDUAL: out is the float32 residual stream, out[t, f] += y[t, f]
//   epilogue TC_SILU_MUL: W alternates 64 gate rows and 64 up rows; out[tokens, features/2] bfloat16
// splits: blocks of a cluster that share the k range (1, 2, 4 or 8; only when tokens <= 64).
LLMRS_API int llmrs_gemm_bf16(const void* x, long long ldx, const void* w, void* out, long long ldo, int tokens,
                              int features, int K, int epilogue, int out_dtype, int splits, int* error_flag,
                              cudaStream_t stream) {
  LLMRS_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_bf16: unknown epilogue %d", epilogue);
  return gemm_bf16_impl(x, ldx, w, out, ldo, tokens, features, K, epilogue, out_dtype, splits, error_flag, nullptr,
                        nullptr, stream);
}

// llmrs_gemm_bf16 as one half of a norm that is spread over two products: with emit_w (TC_RESIDUAL) it also writes emit_xw[tokens, emit_ld] = (h + y) * emit_w in bfloat16 and
// emit_part[pieces, part_stride], the sums of squares per token of each piece of the features (128 wide for at
// most 64 tokens, 256 wide for more); with scale_part it multiplies the rows of y by 1 / sqrt(sum of the
// scale_parts entries of the row's token / scale_dim + scale_eps) before its epilogue.
LLMRS_API int llmrs_gemm_bf16_norm(const void* x, long long ldx, const void* w, void* out, long long ldo, int tokens,
                                   int features, int K, int epilogue, int out_dtype, int splits, const float* emit_w,
                                   void* emit_xw, long long emit_ld, float* emit_part, const float* scale_part,
                                   int part_stride, int scale_parts, int scale_dim, float scale_eps,
                                   int* error_flag, cudaStream_t stream) {
  LLMRS_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_bf16: unknown epilogue %d", epilogue);
  LLMRS_REQUIRE(!emit_w || (epilogue == TC_RESIDUAL && emit_xw && emit_part && part_stride >= tokens),
                "gemm_bf16_norm: the next norm's input is written by a residual epilogue");
  LLMRS_REQUIRE(!emit_w || (((uintptr_t)emit_w & 15) == 0 && ((uintptr_t)emit_xw & 15) == 0 && emit_ld % 8 == 0),
                "gemm_bf16_norm: the norm's weight and input must be 16-byte aligned, rows too");
  LLMRS_REQUIRE(tokens <= 64 || features >= 256, "gemm_bf16_norm: more than 64 tokens need at least 256 features");
  LLMRS_REQUIRE(!scale_part || (scale_parts > 0 && scale_dim > 0 && part_stride >= tokens),
                "gemm_bf16_norm: bad description of the row scales");
  NormLink nl;
  nl.emit_w = emit_w; nl.emit_xw = emit_xw; nl.emit_ld = emit_ld; nl.emit_part = emit_part; nl.scale_part = scale_part;
  nl.part_stride = part_stride; nl.scale_parts = scale_parts; nl.scale_dim = scale_dim; nl.scale_eps = scale_eps;
  return gemm_bf16_impl(x, ldx, w, out, ldo, tokens, features, K, epilogue, out_dtype, splits, error_flag, nullptr, &nl,
                        stream);
}

static int gemm_bf16_impl(const void* x, long long ldx, const void* w, void* out, long long ldo, int tokens,
                          int features, int K, int epilogue, int out_dtype, int splits, int* error_flag,
                          const QkvRope* qr, const NormLink* nl, cudaStream_t stream) {
  LLMRS_REQUIRE(tokens > 0 && features > 0 && K > 0, "gemm_bf16: bad sizes");
  LLMRS_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_bf16: K = %d and the row stride %lld must be multiples of 8", K, ldx);
  LLMRS_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
  LLMRS_REQUIRE(features % 8 == 0 && ldo % 8 == 0, "gemm_bf16: features %d and the output row stride %lld must be "
                "multiples of 8", features, ldo);
  LLMRS_REQUIRE(((uintptr_t)out & 15) == 0, "gemm_bf16: the output must be 16-byte aligned");
  LLMRS_REQUIRE(epilogue != TC_SILU_MUL || features % 128 == 0,
                "gemm_bf16: SiLU*up needs features in groups of 128, got %d", features);
  TcParams p;
  if (qr) p.qr = *qr; else p.qr = QkvRope{};
  const NormLink none;
  const NormLink& L = nl ? *nl : none;
  p.emit_w = L.emit_w; p.emit_xw = (bf16*)L.emit_xw; p.emit_ld = L.emit_ld; p.emit_part = L.emit_part;
  p.scale_part = L.scale_part; p.part_stride = L.part_stride; p.scale_parts = L.scale_parts; p.scale_dim = L.scale_dim;
  p.scale_eps = L.scale_eps;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.k_blocks = (K + TC_BK - 1) / TC_BK; p.error_flag = error_flag;
  p.wait_limit = g_tc_wait_limit; p.test_skip_kb = g_tc_test_skip_kb;
  p.next = llmrs_take_next_prefetch();   // used by the few-token kernel; a many-token launch drops it
  CUtensorMap ma, mb;
  int rc;
  if (tokens <= 64) {
    LLMRS_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_bf16: splits must be 1, 2, 4 or 8");
    const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64;
    if ((rc = make_map(&ma, w, features, K, K, TC_BM))) return rc;
    if ((rc = make_map(&mb, x, tokens, K, ldx, bn))) return rc;
    p.a_rows = features; p.b_rows = tokens;
    dim3 grid((features + TC_BM - 1) / TC_BM, 1, splits);
    // Stages sized so that two blocks fit on an SM: the second one's loads cover the first one's epilogue.
    if (bn == 16) return launch_tc<16, 6, 1>(ma, mb, p, grid, splits, stream);
    if (bn == 32) return launch_tc<32, 5, 1>(ma, mb, p, grid, splits, stream);
    return launch_tc<64, 4, 1>(ma, mb, p, grid, splits, stream);
  }
  const bool wide = features >= 256 || epilogue == TC_SILU_MUL;
  const int bn = wide ? 256 : 128;
  LLMRS_REQUIRE(epilogue != TC_SILU_MUL || features % 256 == 0,
                "gemm_bf16: SiLU*up over many tokens needs features in groups of 256, got %d", features);
  if ((rc = make_map(&ma, x, tokens, K, ldx, TC_BM))) return rc;
  if ((rc = make_map(&mb, w, features, K, K, bn))) return rc;
  p.a_rows = tokens; p.b_rows = features;
  dim3 grid((tokens + TC_BM - 1) / TC_BM, (features + bn - 1) / bn, 1);
  CUtensorMap mh = {};
  if (bn == 256 && epilogue == TC_RESIDUAL && (rc = make_map_h(&mh, out, tokens, features, ldo))) return rc;
  if (bn == 256 && g_tc_pairs && tokens > TC_BM) {
    // Tiles of 256 tokens on pairs of SMs; each block copies its half of a weight tile.
    if ((rc = make_map(&mb, w, features, K, K, PS_BN / 2))) return rc;
    const int n_m = (tokens + 2 * TC_BM - 1) / (2 * TC_BM);
    return launch_pair<2>(ma, mb, mh, p, n_m, n_m * (int)grid.y, nullptr, stream);
  }
  if (bn == 256) return launch_persistent(ma, mb, mh, p, grid.x, grid.x * grid.y, stream);
  return launch_tc<128, 6, 0>(ma, mb, p, grid, 1, stream);
}
