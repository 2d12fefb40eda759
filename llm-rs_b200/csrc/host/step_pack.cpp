// Packing of one step's index arrays for the device (see pack_step in cache_manager.hpp).
//
// The reference reshapes its flat batch to a rectangle (llm-core/src/backends/candle.rs:
// 1122-1125), which is only right when every sequence brings the same number of tokens.
// The batch here is ragged: per token its id, position and request row; per request where
// its tokens start, how many it brings, how many it has cached and its state slot.
#include "cache_manager.hpp"

#include <algorithm>

namespace llmrs_host {

namespace {
int64_t round_up(int64_t n, int64_t m) { return (n + m - 1) / m * m; }
}

bool pack_step(const CacheManager& cm, int n_entries, const int64_t* ids, const int32_t* n_tokens,
               const int32_t* tokens, const int32_t* n_want, const int32_t* want,
               const int32_t* device_token, int table_round,
               int32_t* out, int64_t capacity, int64_t* offsets, int64_t* sizes, int32_t* widths,
               StepShape* shape) {
    if (n_entries < 1) throw Failure{kBadArgument, "a step needs at least one entry"};
    if (table_round < 1) throw Failure{kBadArgument, "table_round must be positive"};
    const int G = cm.n_groups();
    const int R = n_entries;
    std::vector<const Record*> recs(R);
    int64_t T = 0, W = 0;
    for (int r = 0; r < R; ++r) {
        recs[r] = &cm.record(ids[r]);
        int n = n_tokens[r];
        if (n < 1) throw Failure{kBadArgument, "an entry brings no tokens"};
        T += n;
        W += n_want[r];
    }
    for (int g = 0; g < G; ++g) {
        size_t widest = 0;
        for (int r = 0; r < R; ++r) widest = std::max(widest, recs[r]->tables[g].size());
        widths[g] = static_cast<int32_t>(round_up(static_cast<int64_t>(widest), table_round));
    }
    const int n_arrays = kFirstTable + G;
    sizes[kTokenIds] = sizes[kPositions] = sizes[kTokenReq] = T;
    sizes[kQStart] = sizes[kNNew] = sizes[kCachedLen] = sizes[kSlotIds] = R;
    sizes[kWantRows] = W;
    sizes[kPendDst] = sizes[kPendSrc] = R;
    for (int g = 0; g < G; ++g) sizes[kFirstTable + g] = static_cast<int64_t>(R) * widths[g];
    int64_t total = 0;
    for (int a = 0; a < n_arrays; ++a) {
        offsets[a] = total;
        total += round_up(std::max<int64_t>(sizes[a], 1), 4);
    }
    shape->n_tokens = static_cast<int>(T);
    shape->n_requests = R;
    shape->n_want = static_cast<int>(W);
    shape->total = total;
    if (total > capacity || out == nullptr) return false;

    int32_t* token_ids = out + offsets[kTokenIds];
    int32_t* positions = out + offsets[kPositions];
    int32_t* token_req = out + offsets[kTokenReq];
    int32_t* q_start = out + offsets[kQStart];
    int32_t* n_new = out + offsets[kNNew];
    int32_t* cached = out + offsets[kCachedLen];
    int32_t* slots = out + offsets[kSlotIds];
    int32_t* want_rows = out + offsets[kWantRows];
    int32_t* pend_dst = out + offsets[kPendDst];
    int32_t* pend_src = out + offsets[kPendSrc];
    int64_t at = 0, w_at = 0, want_in = 0;
    for (int r = 0; r < R; ++r) {
        const Record& rec = *recs[r];
        int n = n_tokens[r];
        for (int i = 0; i < n; ++i) {
            token_ids[at + i] = tokens[at + i];
            positions[at + i] = rec.cached_len + i;
            token_req[at + i] = r;
        }
        q_start[r] = static_cast<int32_t>(at);
        n_new[r] = n;
        cached[r] = rec.cached_len;
        slots[r] = rec.slot;
        for (int i = 0; i < n_want[r]; ++i) {
            int w = want[want_in + i];
            if (w < 0 || w >= n) throw Failure{kBadArgument, "a wanted place lies outside its entry's tokens"};
            want_rows[w_at++] = static_cast<int32_t>(at + w);
        }
        want_in += n_want[r];
        if (device_token != nullptr && device_token[r] >= 0) {
            // The entry's single token is still on the device: a kernel copies it in.
            pend_dst[r] = static_cast<int32_t>(at);
            pend_src[r] = device_token[r];
            token_ids[at] = 0;
        } else {
            pend_dst[r] = -1;
            pend_src[r] = 0;
        }
        at += n;
    }
    for (int g = 0; g < G; ++g) {
        int32_t* tab = out + offsets[kFirstTable + g];
        const int width = widths[g];
        for (int r = 0; r < R; ++r) {
            const auto& table = recs[r]->tables[g];
            int32_t* row = tab + static_cast<int64_t>(r) * width;
            std::copy(table.begin(), table.end(), row);
            std::fill(row + table.size(), row + width, kReleased);
        }
    }
    return true;
}

bool plan_paged_attention(int n_requests, const int32_t* n_new, const int32_t* cached_len, int tile,
                          int32_t* tiles_out, int64_t tiles_capacity, int32_t* decode_out,
                          int64_t decode_capacity, AttentionPlan* plan) {
    if (n_requests < 0 || tile < 1) throw Failure{kBadArgument, "attention plan: bad sizes"};
    int64_t tiles = 0, dec = 0, long_blocks = 0, long_tokens = 0;
    int max_dec_kv = 0;
    for (int r = 0; r < n_requests; ++r) {
        const int n = n_new[r];
        if (n == 1) {
            ++dec;
            max_dec_kv = std::max(max_dec_kv, cached_len[r] + 1);
        } else if (n > 1) {
            tiles += (n + tile - 1) / tile;
            long_blocks += (n + 127) / 128;
            long_tokens += n;
        }
    }
    plan->n_tiles = static_cast<int>(tiles);
    plan->n_decode = static_cast<int>(dec);
    plan->max_decode_kv_len = max_dec_kv;
    // Blocks of 128 queries pay off when the portions fill them at least half on average.
    plan->long_portions = long_blocks > 0 && long_tokens >= 64 * long_blocks;
    if (tiles > tiles_capacity || dec > decode_capacity) return false;
    int64_t t_at = 0, d_at = 0;
    for (int r = 0; r < n_requests; ++r) {
        const int n = n_new[r];
        if (n == 1) {
            decode_out[d_at++] = r;
        } else {
            for (int off = 0; off < n; off += tile) {
                tiles_out[t_at++] = r;
                tiles_out[t_at++] = off;
            }
        }
    }
    return true;
}

}  // namespace llmrs_host
