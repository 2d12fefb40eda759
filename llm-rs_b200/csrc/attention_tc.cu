// Prefill attention on tcgen05 for head_dim 128, bfloat16, pages of a multiple of 16 keys.
//
// A block owns 128 query tokens of one request and one query head; its thread r owns
// query row r, which is lane r of tensor memory, so the softmax needs no exchange
// between threads. Shared memory feeds the tensor cores at roughly 64 bytes a cycle, less
// than two operands of an MMA want, so the left operand of both products lives in tensor
// memory and shared memory holds only K and V. Per tile of 64 keys:
//   S = Q K^T   tcgen05.mma, 128x64x128; Q sits in tensor memory (each thread put its row
//               there once), K in shared memory (TMA, 128-byte swizzle); S goes to tensor
//               memory (64 columns of float32);
//   softmax     every thread reads its row of S (tcgen05.ld), masks it if the tile touches
//               the diagonal or the window's edge, and writes P = 2^(s*c - m) as bfloat16
//               pairs over the first 32 columns of S (tcgen05.st). The reference maximum m
//               of a row only moves when the row's maximum grew by more than 8 (a factor
//               256): then, and only then, the row of O in tensor memory is rescaled
//               (tcgen05.ld, multiply, tcgen05.st);
//   O += P V    tcgen05.mma, 128x128x64; P is read from tensor memory, V is used as it lies
//               in its pages (keys x head_dim, MN-major operand).
// A fifth warp issues the MMAs and a sixth the TMA copies (one box per page, or per 64 keys of
// a larger page, and half of the head; the boxes of a tile are issued by as many lanes side by
// side, since one copy costs its issuer some 80 cycles), so the softmax threads never wait for
// issue work and the copies never delay an MMA. K and V go through a ring of three stages. The
// roles meet at mbarriers only. A block holds all 512 columns of tensor memory (S twice, O, Q), so one
// block runs per SM; S of the next tile is computed while the softmax of this one runs. Blocks with the
// longest rows of keys are scheduled first.
//
// Same contract and math as attn_prefill_kernel in attention.cu (scores, softmax and the
// weighted sum accumulate in float32; llm-core/src/backends/candle.rs:1587-1640). Every
// wait is bounded (llmrs_attention_tc_set_wait_limit polls, 2^22 by default); when one runs out
// the block raises a flag in its shared memory at which all its roles leave their loops, waits
// (bounded) for its copies and MMAs in flight, records the error, stores nothing and frees its
// tensor memory.
#include <cuda.h>
#include <mutex>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

namespace {

constexpr int AT_BQ = 128, AT_BK = 128, AT_D = 128, AT_THREADS = 128, AT_STAGES = 3;
constexpr uint32_t AT_WAIT_LIMIT = 1u << 22;
constexpr int AT_MAX_LIST = 8192;    // entries of the tile list that a launch takes (a block notes its 128-row tiles in shared memory)
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr uint32_t K_BYTES = AT_BK * AT_D * 2, V_BYTES = K_BYTES, STAGE_BYTES = K_BYTES + V_BYTES;
constexpr uint32_t HALF_BYTES = AT_BK * 128;   // one half of head_dim of a K or V tile: [128 keys][64 dims]
// Tensor memory of a block: S twice (128 columns of float32 each; P, as bfloat16 pairs, goes over the
// first 64 of its S), O (128 columns), Q (128 bfloat16 = 64 columns).
constexpr uint32_t TMEM_COLS = 512, S_COL = 0, O_COL = 256, Q_COL = 384;

__device__ int g_attn_tc_error = 0;

__device__ __forceinline__ uint32_t sm(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar)); }
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, uint32_t limit, volatile int* abort_flag) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (bar_try(bar, parity)) return true;
    if (it > 128) {
      __nanosleep(32);
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}
// Bounded wait of a block that has given up already, for what it still has in flight: the flag does not cut it short.
__device__ __forceinline__ void bar_drain(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (bar_try(bar, parity)) return;
    if (it > 128) __nanosleep(32);
  }
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle. K-major operands: lbo unused (1),
// sbo = 1024 (8 rows of 128 bytes). MN-major operands: lbo = distance between blocks of 64
// elements along MN, sbo = distance between groups of 8 rows along K.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> f32, M = 128, N = n; b_mn: the B operand is MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// D (+)= A B with A in tensor memory (lane = row, two bfloat16 per column, 8 columns per k16 step)
// and B described in shared memory.
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t leader;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(leader));
  return leader != 0;
}
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive float32 columns of this thread's lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void bar_init_n(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Threads 0..127 (warps 0-3) are the softmax threads: thread r owns query row r. One lane of warp 4
// issues every MMA, the lanes of warp 5 the TMA copies. Nobody meets at a block-wide barrier inside
// the loop; the roles talk through mbarriers:
//   q              all 128 threads have put their query rows into tensor memory
//   kfull[3]       K of a tile has landed in its slot (TMA bytes); vfull[3] the same for V
//   kfree[3]       the MMAs of S that read the slot are done (tcgen05.commit); vfree[3]: those of O += P V
//   s[2]           S of a tile is in its buffer of tensor memory
//   p[2]           all 128 threads have written P of a tile over its S
//   o[2]           O += P V of a tile is done
// Barriers that are used every tile come in pairs, one per parity of the tile: the roles run up to
// two tiles apart, and a wait by parity must never be a whole phase behind its barrier.
__global__ void __launch_bounds__(AT_THREADS + 96, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, long long q_stride,
                       bf16* __restrict__ out, long long out_stride, const int* __restrict__ tiles,
                       const int* __restrict__ q_start, const int* __restrict__ n_new,
                       const int* __restrict__ cached_len, const int* __restrict__ block_table, int table_stride,
                       int n_list, int persistent, int n_q_heads, int n_kv_heads, int page_size, int box_rows, int window, float scale,
                       int* __restrict__ error_flag, uint32_t wait_limit, int test_skip_tile) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = smem_raw;           // 1024-byte aligned (checked below): the swizzle pattern needs it
  unsigned char* KV = base;                 // AT_STAGES x (K: 2 halves of [64 keys][64 dims], then V the same)
  uint64_t* bars = reinterpret_cast<uint64_t*>(KV + AT_STAGES * STAGE_BYTES);   // kfull[3], kfree[3], vfull[3], vfree[3], s[2], p[2], o[2], q, drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * AT_STAGES + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_valid_slot = reinterpret_cast<int*>(tmem_slot + 2);
  uint16_t* valid = reinterpret_cast<uint16_t*>(tmem_slot + 4);     // AT_MAX_LIST entries: the list's 128-row tiles

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((sm(base) & 1023u) != 0) {            // never seen; without the alignment the operands would be garbage
    if (threadIdx.x == 0) atomicExch(error_flag ? error_flag : &g_attn_tc_error, 3);
    return;
  }
  // The work: an item is 128 query rows of one request and one query head: those entries of the list of 64-query
  // tiles whose offset is a multiple of 128 (warp 0 notes them in shared memory first), times the heads. Items are
  // numbered so that later tiles of a prompt, which see more keys, come first, for every head; block b of G walks
  // the numbering like a snake (b, 2G-1-b, 2G+b, 4G-1-b, ...), which gives every block about the same number of
  // key tiles, and keeps tensor memory, barriers and the ring of stages from one item to the next: the copies of an
  // item's first keys run under the end of the item before.
  // With a block per item (persistent == 0) the block's number names an entry and a head, and the block of an entry
  // that starts no 128-row tile leaves at once.
  if (!persistent && tiles[2 * (n_list - 1 - (int)blockIdx.x / n_q_heads) + 1] % AT_BQ != 0) return;
  if (persistent && warp == 0) {
    int n = 0;
    for (int e0 = 0; e0 < n_list; e0 += 32) {
      const int e = e0 + lane;
      const bool is_item = e < n_list && tiles[2 * e + 1] % AT_BQ == 0;
      const unsigned m = __ballot_sync(0xffffffffu, is_item);
      if (is_item) valid[n + __popc(m & ((1u << lane) - 1u))] = (uint16_t)e;
      n += __popc(m);
    }
    if (lane == 0) *n_valid_slot = n;
  }
  __syncthreads();
  const int n_valid = persistent ? *n_valid_slot : n_list;
  struct Item {
    int rows, tok0, pos0, kv_hi, key_floor, kv_lo, n_tiles, head, kvh;
    const int* table;
  };
  const int n_lin = n_valid * n_q_heads;
  auto item_index = [&](int r) {    // the block's r-th item, or -1 when it has no more
    if (!persistent) return r == 0 ? (int)blockIdx.x : -1;
    const int G = (int)gridDim.x, b = (int)blockIdx.x;
    const int L = (r & 1) ? (r + 1) * G - 1 - b : r * G + b;
    return L < n_lin ? L : -1;
  };
  auto item_at = [&](int L, Item& it) {
    const int e = n_valid - 1 - L / n_q_heads, tile = persistent ? (int)valid[e] : e;
    const int req = tiles[2 * tile], q_off = tiles[2 * tile + 1];
    it.head = L % n_q_heads;
    it.kvh = it.head / (n_q_heads / n_kv_heads);
    it.rows = min(AT_BQ, n_new[req] - q_off);
    it.tok0 = q_start[req] + q_off;
    it.pos0 = cached_len[req] + q_off;
    it.kv_hi = it.pos0 + it.rows;
    it.key_floor = window > 0 ? max(0, it.pos0 - window + 1) : 0;
    it.kv_lo = (it.key_floor / AT_BK) * AT_BK;
    it.n_tiles = (it.kv_hi - it.kv_lo + AT_BK - 1) / AT_BK;
    it.table = block_table + (size_t)req * table_stride;
    return true;
  };
  if (item_index(0) < 0) return;     // more blocks than items

  const uint32_t bar_kfull = sm(bars), bar_kfree = sm(bars + AT_STAGES), bar_vfull = sm(bars + 2 * AT_STAGES),
                 bar_vfree = sm(bars + 3 * AT_STAGES), bar_s = sm(bars + 4 * AT_STAGES), bar_p = bar_s + 16,
                 bar_o = bar_s + 32, bar_q = bar_s + 48, bar_drain_mma = bar_s + 56;
  if (tid == 0) {
    for (int i = 0; i < 4 * AT_STAGES + 2; ++i) bar_init(sm(bars + i));
    bar_init_n(bar_p, AT_THREADS);
    bar_init_n(bar_p + 8, AT_THREADS);
    bar_init(bar_o);
    bar_init(bar_o + 8);
    bar_init_n(bar_q, AT_THREADS);
    bar_init(bar_drain_mma);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t idesc_s = instr_desc(AT_BK, 0), idesc_pv = instr_desc(AT_D, 1);

  int copies = 0;   // copying warps: tiles (counted over the block's items) whose copies the warp has requested
  auto wait_all = [&](uint32_t bar, uint32_t parity) {
    return __all_sync(0xffffffffu, bar_wait(bar, parity, wait_limit, abort_flag));
  };
  // Every role walks the block's items in the same order and counts their key tiles on: `g0` is the number of
  // tiles of the items before, and tile t of an item uses the stage (g0 + t) % 3 and the barriers' phases of g0 + t.
  if (warp >= 5) {
    // ---- the copying warps: warp 5 brings K, warp 6 V; one box per lane, and a lane's box of tile t
    // is the same part of every tile.
    const int which = warp - 5;
    const int per_half = AT_BK / box_rows;            // boxes per half of the head: 8 or 2
    const int n_boxes = 2 * per_half;
    const int h = lane / per_half, i = lane % per_half;
    const uint32_t box_bytes = (uint32_t)box_rows * 128;
    const uint32_t bar_full = which ? bar_vfull : bar_kfull, bar_free = which ? bar_vfree : bar_kfree;
    int g0 = 0;
    bool ok = true;
    for (int r = 0; ok; ++r) {
      const int L = item_index(r);
      if (L < 0) break;
      Item it;
      item_at(L, it);
      // Page of this lane's box of tile t, or -1 (the lane copies nothing). A box whose keys no query of
      // the item may see (past the end, or before the window) is filled from the page of the newest key
      // instead: whatever a slot holds must be finite (it meets a probability of zero), and shared memory
      // that no copy ever wrote need not be.
      const int spare_page = LLMRS_CHECKED_PAGE(it.table[(it.kv_hi - 1) / page_size], 6, it.kv_hi - 1);
      auto page_of = [&](int t) {
        const int key = it.kv_lo + t * AT_BK + box_rows * i;
        if (lane >= n_boxes || t >= it.n_tiles) return -1;
        return (key < it.kv_hi && key + box_rows - 1 >= it.key_floor) ? LLMRS_CHECKED_PAGE(it.table[key / page_size], 6, key)
                                                                     : spare_page;
      };
      int page = page_of(0);                          // looked up one tile ahead of its copy
      for (int t = 0; t < it.n_tiles; ++t) {
        const int g = g0 + t, st = g % AT_STAGES;
        const int next = page_of(t + 1);
        // The stage is free once the MMAs that read the tile three before are done.
        if (g >= AT_STAGES && !wait_all(bar_free + 8 * st, ((g / AT_STAGES) - 1) & 1)) { ok = false; break; }
        copies = g + 1;
        if (!(which == 0 && g == test_skip_tile)) {   // tests only: K of this tile never arrives
          const unsigned live = __ballot_sync(0xffffffffu, page >= 0);
          const uint32_t bar = bar_full + 8 * st;
          if (lane == 0) bar_expect(bar, (uint32_t)__popc(live) * box_bytes);
          __syncwarp();
          if (page >= 0) {
            const int key = it.kv_lo + t * AT_BK + box_rows * i;
            const int row = ((page * n_kv_heads + it.kvh) * 2 + which) * page_size + key % page_size;
            tma_2d(sm(KV) + st * STAGE_BYTES + which * K_BYTES + h * HALF_BYTES + i * box_bytes, &map_kv, bar, h * 64, row);
          }
          __syncwarp();
        }
        page = next;
      }
      g0 += it.n_tiles;
    }
  } else if (warp == 4) {
    // ---- the MMA warp: all lanes walk the loop together; lane 0 issues -------------------------
    // One elected lane issues, but the whole warp computes the operands of every MMA: they are then
    // the same in all lanes, which lets the compiler keep them in uniform registers, where the MMA
    // wants them. Issued from a divergent branch (`if (lane == 0)`) an MMA of this size costs its
    // thread some 120 cycles instead of the 32 to 64 that the tensor cores need for it.
    const bool leader = elect_one();
    auto issue_s = [&](int g) {     // S of the tile with running number g = Q K^T into S buffer g % 2; Q is read from tensor memory
      const uint32_t kbuf = sm(KV) + (g % AT_STAGES) * STAGE_BYTES;
      const uint32_t s_col = tmem + S_COL + (g & 1) * AT_BK;
#pragma unroll
      for (int kk = 0; kk < AT_D / 16; ++kk) {
        const uint32_t half = kk / 4;   // head_dim 0-63 or 64-127: each half is its own swizzled tile
        const uint64_t bd = smem_desc(kbuf + half * HALF_BYTES + (kk % 4) * 32, 16, 1024);
        if (leader) mma_ts(s_col, tmem + Q_COL + kk * 8, bd, idesc_s, kk > 0 ? 1u : 0u);
      }
      if (leader) {
        commit(bar_s + 8 * (g & 1));
        commit(bar_kfree + 8 * (g % AT_STAGES));   // the slot of K may be refilled
      }
      __syncwarp();
    };
    int g0 = 0, n_done = 0;
    bool ok = true;
    for (int r = 0; ok; ++r) {
      const int L = item_index(r);
      if (L < 0) break;
      Item it;
      item_at(L, it);
      const int n_tiles = it.n_tiles;
      // S runs one tile ahead of the softmax: S of tiles 0 and 1 now (the item's queries are in tensor memory,
      // which also says that the softmax threads are done with the item before), S of tile j+2 as soon as P of
      // tile j (which lies over S of tile j) has been used.
      ok = wait_all(bar_q, n_done & 1) && wait_all(bar_kfull + 8 * (g0 % AT_STAGES), (g0 / AT_STAGES) & 1);
      if (ok) {
        fence_after();
        issue_s(g0);
      }
      if (ok && n_tiles > 1) {
        ok = wait_all(bar_kfull + 8 * ((g0 + 1) % AT_STAGES), ((g0 + 1) / AT_STAGES) & 1);
        if (ok) {
          fence_after();
          issue_s(g0 + 1);
        }
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = g0 + j, st = g % AT_STAGES;
        // K of tile j+2 has landed long before P of tile j is there: look before the wait that matters.
        if (j + 2 < n_tiles) {
          ok = wait_all(bar_kfull + 8 * ((g + 2) % AT_STAGES), ((g + 2) / AT_STAGES) & 1);
          if (!ok) break;
        }
        // O += P V of tile j: its V has landed, and P is written.
        ok = wait_all(bar_vfull + 8 * st, (g / AT_STAGES) & 1) && wait_all(bar_p + 8 * (g & 1), (g >> 1) & 1);
        if (!ok) break;
        fence_after();
        {
          const uint32_t vbuf = sm(KV) + st * STAGE_BYTES + K_BYTES;
          const uint32_t p_col = tmem + S_COL + (g & 1) * AT_BK;
#pragma unroll
          for (int kk = 0; kk < AT_BK / 16; ++kk) {
            const uint64_t bd = smem_desc(vbuf + kk * 2048, HALF_BYTES, 1024);
            if (leader) mma_ts(tmem + O_COL, p_col + kk * 8, bd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
          if (leader) {
            commit(bar_vfree + 8 * st);  // the slot of V may be refilled
            commit(bar_o + 8 * (g & 1)); // O holds the item's tiles 0..j
          }
        }
        __syncwarp();
        // S of tile j+2 goes over P of tile j: the tensor cores run MMAs in the order of issue.
        if (j + 2 < n_tiles) issue_s(g + 2);
      }
      g0 += n_tiles;
      ++n_done;
    }
  } else {
    // ---- softmax threads ------------------------------------------------------------------
    const int row = tid;                      // this thread's query row = its lane of tensor memory
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    const float sl2 = scale * AT_LOG2E;
    int g0 = 0;
    bool ok = true;
    for (int r = 0; ok; ++r) {
      const int L = item_index(r);
      if (L < 0) break;
      Item it;
      item_at(L, it);
      const int n_tiles = it.n_tiles, pos0 = it.pos0, rows = it.rows;
      // The query row goes into tensor memory (two bfloat16 per column), where Q K^T reads it as its
      // A operand: shared memory then only has to feed K. (Every MMA of the item before is done: this thread
      // has waited for its last O.)
      {
        const uint4* qrow = reinterpret_cast<const uint4*>(q + (size_t)(it.tok0 + row) * q_stride + (size_t)it.head * AT_D);
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t rr[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = row < rows ? qrow[hlf * 8 + c] : make_uint4(0u, 0u, 0u, 0u);
            rr[4 * c] = v.x; rr[4 * c + 1] = v.y; rr[4 * c + 2] = v.z; rr[4 * c + 3] = v.w;
          }
          tmem_st32u(lane_addr + Q_COL + hlf * 32, rr);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        fence_before();
        bar_arrive(bar_q);
      }
      const int my_pos = pos0 + row;
      float m_ref = -INFINITY, l_sum = 0.f;
      for (int j = 0; j < n_tiles; ++j) {
        const int g = g0 + j;
        const int kb = it.kv_lo + j * AT_BK;
        const uint32_t s_addr = lane_addr + S_COL + (g & 1) * AT_BK;
        ok = __all_sync(0xffffffffu, bar_wait(bar_s + 8 * (g & 1), (g >> 1) & 1, wait_limit, abort_flag));
        if (!ok) break;
        fence_after();
        // This thread's 128 scores -> probabilities.
        float s[AT_BK];
#pragma unroll
        for (int c = 0; c < AT_BK; c += 32) {
          float t0[32];
          tmem_ld32(s_addr + c, t0);
#pragma unroll
          for (int e = 0; e < 32; ++e) s[c + e] = t0[e];
        }
        const bool need_mask = kb + AT_BK - 1 > pos0 || (window > 0 && kb <= pos0 + AT_BQ - 1 - window);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < AT_BK; ++c) {
            const int key = kb + c;
            const bool seen = key <= my_pos && (window <= 0 || key > my_pos - window);
            s[c] = seen ? s[c] : -INFINITY;
          }
        }
        // Four running maxima (and sums below): a chain of 128 dependent operations would be the
        // longest thing this thread does.
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < AT_BK; c += 4) {
          mx4[0] = fmaxf(mx4[0], s[c]); mx4[1] = fmaxf(mx4[1], s[c + 1]);
          mx4[2] = fmaxf(mx4[2], s[c + 2]); mx4[3] = fmaxf(mx4[3], s[c + 3]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // The reference maximum moves only when the row's maximum outgrew it by a factor 256.
        const float m_tile = mx * sl2;
        float factor = 1.f;
        bool moved = false;
        if (m_tile > m_ref + 8.f) {   // also the first tile with a visible key (m_ref = -inf)
          factor = m_ref == -INFINITY ? 0.f : ex2(m_ref - m_tile);
          m_ref = m_tile;
          moved = j > 0;
          l_sum *= factor;
        }
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        // P goes over S (all of this thread's S is in registers by now), 64 keys at a time.
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c0 = 0; c0 < AT_BK / 2; c0 += 32) {
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float p0 = ex2(fmaf(s[2 * (c0 + c)], sl2, -m_use));
            const float p1 = ex2(fmaf(s[2 * (c0 + c) + 1], sl2, -m_use));
            sum4[c & 3] += p0 + p1;
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
            pk[c] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          tmem_st32u(s_addr + c0, pk);
        }
        l_sum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        // Where a row's reference moved, O is rescaled (rare after the first tiles; the loads and
        // stores of tensor memory are warp-wide, so the warp decides together), once O += P V of the
        // tile before is done (S of tile j implies O += P V of tile j-2 only).
        if (__any_sync(0xffffffffu, moved)) {
          ok = __all_sync(0xffffffffu, bar_wait(bar_o + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, wait_limit, abort_flag));
          if (!ok) break;
          fence_after();
#pragma unroll 1
          for (int c = 0; c < AT_D; c += 32) {
            float o[32];
            tmem_ld32(lane_addr + O_COL + c, o);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] *= factor;
            tmem_st32(lane_addr + O_COL + c, o);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        fence_before();
        bar_arrive(bar_p + 8 * (g & 1));
      }
      const int g_last = g0 + n_tiles - 1;
      if (ok) ok = __all_sync(0xffffffffu, bar_wait(bar_o + 8 * (g_last & 1), (g_last >> 1) & 1, wait_limit, abort_flag));
      fence_after();
      if (ok) {
        // Every thread reads its row of O (the load is warp-wide); rows past the portion's end are not stored.
        const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
        bf16* orow = out + (size_t)(it.tok0 + row) * out_stride + (size_t)it.head * AT_D;
#pragma unroll 1
        for (int c = 0; c < AT_D; c += 32) {
          float o[32];
          tmem_ld32(lane_addr + O_COL + c, o);
          if (row < rows) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 pk;
              __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int q8 = 0; q8 < 4; ++q8) h2[q8] = __floats2bfloat162_rn(o[e + 2 * q8] * inv, o[e + 2 * q8 + 1] * inv);
              *reinterpret_cast<uint4*>(orow + c + e) = pk;
            }
          }
          __syncwarp();
        }
      }
      g0 += n_tiles;
    }
  }
  fence_before();
  __syncthreads();
  if (*abort_flag) {
    // The block gave up. Before tensor memory is freed and the block leaves: the MMAs that were issued must be
    // done, and no copy may still be on its way into this block's shared memory.
    if (warp == 4) {
      if (elect_one()) commit(bar_drain_mma);
      __syncwarp();
      bar_drain(bar_drain_mma, 0, wait_limit);
    } else if (warp >= 5) {
      const int which = warp - 5;
      const uint32_t bar_full = which ? bar_vfull : bar_kfull;
      for (int t = max(0, copies - AT_STAGES); t < copies; ++t)
        if (!(which == 0 && t == test_skip_tile)) bar_drain(bar_full + 8 * (t % AT_STAGES), (t / AT_STAGES) & 1, wait_limit);
    } else if (tid == 0) {
      atomicExch(error_flag ? error_flag : &g_attn_tc_error, 2);
    }
  }
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
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

int make_map(CUtensorMap* map, const void* basep, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return llmrs_fail("attn_prefill_tc: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(basep), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return llmrs_fail("attn_prefill_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

uint32_t g_wait_limit = AT_WAIT_LIMIT;
int g_test_skip_tile = -1;

}  // namespace

// Polls of a barrier before a wait of the tcgen05 prefill kernel gives up (0: the default, 2^22).
LLMRS_API void llmrs_attention_tc_set_wait_limit(unsigned polls) { g_wait_limit = polls ? polls : AT_WAIT_LIMIT; }

// For the test of the bounded waits only: the next launches never copy K of their tile with this index, so that a
// wait of every block runs out (-1, the default: every copy is made).
LLMRS_API void llmrs_attention_tc_test_skip_copy(int tile) { g_test_skip_tile = tile; }

// Non-zero if a block of the tcgen05 prefill kernel that was launched without an error word of the caller's
// gave up on a wait since the last call (clears the flag).
LLMRS_API int llmrs_attention_tc_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
  return v;
}

// True when llmrs_attn_prefill_tc can take this problem.
bool llmrs_attn_prefill_tc_supported(const void* q, long long q_stride, const void* cache, int d, int page_size,
                                     float scale) {
  return d == AT_D && page_size % 16 == 0 && scale > 0.f && q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 &&
         ((uintptr_t)cache & 15) == 0 && encode_tiled() != nullptr;
}

// Prefill attention on tcgen05 (see the head of this file). `n_tokens` is the number of rows of q,
// `cache_rows` = n_pages * n_kv_heads * 2 * page_size the number of head_dim-wide rows of the cache.
int llmrs_attn_prefill_tc(const void* q, long long q_stride, int n_tokens, void* out, long long out_stride,
                          const void* cache, long long cache_rows, const int* tiles, int n_tiles, const int* q_start,
                          const int* n_new, const int* cached_len, const int* block_table, int table_stride,
                          int n_q_heads, int n_kv_heads, int page_size, int window, float scale, int* error_flag,
                          cudaStream_t stream) {
  CUtensorMap map_kv;
  int rc;
  (void)n_tokens;
  // One copy per page and half of the head; a page of a multiple of 64 keys is copied 64 keys at a time.
  const int box_rows = page_size % 64 == 0 ? 64 : 16;
  if ((rc = make_map(&map_kv, cache, cache_rows, AT_D, AT_D, box_rows))) return rc;
  const size_t smem = AT_STAGES * STAGE_BYTES + (4 * AT_STAGES + 8) * 8 + 16 + 2 * AT_MAX_LIST;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_prefill_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  // A block holds all of tensor memory, so an SM runs one at a time. With up to 16 items per SM one block per SM
  // walks its share of them, and an item's start runs under the end of the item before (one prompt of 1,024 /
  // 2,048 / 4,096 / 8,192 tokens: 27 / 62 / 173 / 589 us against 30 / 69 / 183 / 595 with a block per item). With
  // more, a block per item, which the hardware hands out longest first: fixed shares then lose more than the
  // starts cost (32,768 tokens: 8.8 against 8.55 ms).
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (n_sm <= 0) n_sm = 1;
  }
  // (About every second entry of the list starts a 128-row tile; a block that finds no item leaves at once.)
  const long long n_lin = (long long)n_q_heads * n_tiles, n_items = (long long)n_q_heads * ((n_tiles + 1) / 2);
  const int persistent = n_items > n_sm && n_items <= 16LL * n_sm ? 1 : 0;
  dim3 grid((unsigned)(persistent ? n_sm : n_lin));
  attn_prefill_tc_kernel<<<grid, AT_THREADS + 96, smem, stream>>>(map_kv, (const bf16*)q, q_stride, (bf16*)out, out_stride,
                                                              tiles, q_start, n_new, cached_len, block_table,
                                                              table_stride, n_tiles, persistent, n_q_heads, n_kv_heads, page_size,
                                                              box_rows, window, scale, error_flag, g_wait_limit,
                                                              g_test_skip_tile);
  return llmrs_launch_status("attn_prefill_tc");
}
