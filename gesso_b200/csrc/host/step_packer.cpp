// One step's metadata, checked, reserved and packed on the host in a single call.
//
// A step is a list of segments: (request, its next tokens, the places among them whose logits are
// wanted).  The device reads the step from one int32 buffer; WHERE each field lies in that buffer is
// decided in one place only, the layout table of the Python side (engine/batch.py: StepLayout), which
// hands the offsets down as an array indexed by the field numbers below.  This file knows what goes
// INTO a field, not where the field is, so a field added to the table moves nothing here.
//
// The cache manager (cache_manager.cpp) is used through its C interface only: it reserves pages for all
// the step's requests or for none and lends its block-table rows; it knows nothing of this buffer.
//
// Stand-in segments (request handle 0) fill a step up to a shape whose CUDA graph exists: they sit on a
// scratch state slot and scratch cache pages that no request owns, start at position 0 and bring token
// id 0; to the kernels they are ordinary segments.
#include <cstdint>
#include <cstring>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

extern "C" {
int gesso_cm_reserve_step(void* cm, const int64_t* rids, const int* n_new, int n, int* starts, int* slots,
                          int* fresh_slots, int* info);
const int* gesso_cm_row(void* cm, int64_t rid, int group, int* n_used);
}

namespace {

// field numbers: the order of the core fields in the layout table (engine/batch.py: CORE_FIELDS)
enum Field {
    F_TOKEN_IDS = 0,   // [tokens]   token ids
    F_POSITIONS,       // [tokens]   absolute position of every token
    F_SEG_OF_TOKEN,    // [tokens]   segment of every token
    F_SEG_START,       // [segs + 1] first token of every segment, and the total
    F_SEG_POS0,        // [segs]     position of a segment's first token
    F_SLOTS,           // [segs]     state slot of a segment's request
    F_LOGIT_ROWS,      // [rows]     tokens whose logits are wanted
    F_TILE_SEG,        // [tiles]    the step's query tiles: segment ...
    F_TILE_Q0,         // [tiles]    ... and first token inside the segment
    F_KV_SPAN,         // [2]        the longest sequence after the step and the average one, over the real requests
    F_BLOCK_TABLE0,    // [segs][max_pages] per paged group g: field F_BLOCK_TABLE0 + g
};

enum {
    OK = 0,
    E_BAD_ARG = -6,        // sizes that do not fit the layout (a bug of the caller)
    E_TWICE = -20,         // a request appears twice (info[4] = segment)
    E_EMPTY_SEG = -21,     // a segment without tokens (info[4] = segment)
    E_TOKEN = -22,         // a token id outside the vocabulary (info[4] = segment, info[5] = the id)
    E_WANT = -23,          // a wanted place outside the segment (info[4] = segment, info[5] = the place)
};

}  // namespace

// rids[n]:       request handles, 0 for a stand-in segment
// n_new[n]:      tokens of every segment (>= 1)
// tokens:        all token ids, segment after segment (sum of n_new), or null: the ids are filled in later
// want_n[n], want: wanted places of every segment (indices into its own tokens), segment after segment
// off[n_off]:    offsets of the fields, by field number; n_off = F_BLOCK_TABLE0 + groups
// sizes[4]:      the layout's capacity: tokens, segments, rows, tiles (a padded step may not use all tiles:
//                the rest repeat the first tile of the last segment; rows must be used up exactly)
// scratch[1+G]:  scratch slot, then the scratch page of every group (used by stand-ins)
// info[8] out:   [0] fresh slots, [1] longest sequence after the step, [2] rows written, [3] tiles used,
//                [4], [5] details of an error
// Returns 0, one of the codes above, or the cache manager's code (nothing was reserved then).
HOST_API int gesso_step_prepare(void* cm, const int64_t* rids, const int* n_new, int n, const int* tokens,
                                const int* want_n, const int* want, const int* off, int n_off, const int* sizes,
                                int groups, int max_pages, int query_tile, int vocab, const int* scratch, int* out,
                                int out_cap, int* fresh_slots, int* info) {
    if (n <= 0 || n_off != F_BLOCK_TABLE0 + groups || query_tile <= 0) return E_BAD_ARG;
    const int cap_tokens = sizes[0], cap_segs = sizes[1], cap_rows = sizes[2], cap_tiles = sizes[3];
    if (n != cap_segs) return E_BAD_ARG;
    // ---- checks: nothing is reserved or written before they all pass ----
    long long total = 0, rows_total = 0, tiles_total = 0;
    std::vector<int64_t> real_rids;
    std::vector<int> real_new, real_at;
    {
        const int* tp = tokens;
        const int* wp = want;
        for (int i = 0; i < n; ++i) {
            const int k = n_new[i];
            if (k < 1) { info[4] = i; return E_EMPTY_SEG; }
            if (rids[i] != 0) {
                for (size_t j = 0; j < real_rids.size(); ++j)
                    if (real_rids[j] == rids[i]) { info[4] = i; return E_TWICE; }
                real_rids.push_back(rids[i]);
                real_new.push_back(k);
                real_at.push_back(i);
            }
            if (tokens) {
                for (int t = 0; t < k; ++t)
                    if (tp[t] < 0 || tp[t] >= vocab) { info[4] = i; info[5] = tp[t]; return E_TOKEN; }
                tp += k;
            }
            for (int w = 0; w < want_n[i]; ++w)
                if (wp[w] < 0 || wp[w] >= k) { info[4] = i; info[5] = wp[w]; return E_WANT; }
            wp += want_n[i];
            total += k;
            rows_total += want_n[i];
            tiles_total += (k + query_tile - 1) / query_tile;
        }
    }
    if (total != cap_tokens || rows_total != cap_rows || tiles_total > cap_tiles) return E_BAD_ARG;
    for (int f = 0; f < n_off; ++f)
        if (off[f] < 0 || off[f] > out_cap) return E_BAD_ARG;
    // ---- pages for every real request, or for none ----
    const int n_real = (int)real_rids.size();
    std::vector<int> starts(n_real > 0 ? n_real : 1), slots(n_real > 0 ? n_real : 1);
    int cm_info[4] = {0, 0, 0, 0};
    if (n_real > 0) {
        const int e = gesso_cm_reserve_step(cm, real_rids.data(), real_new.data(), n_real, starts.data(), slots.data(),
                                            fresh_slots, cm_info);
        if (e != OK) {
            info[4] = (cm_info[0] >= 0 && cm_info[0] < n_real) ? real_at[cm_info[0]] : 0;
            return e;
        }
    }
    // ---- fill the fields ----
    int* tok = out + off[F_TOKEN_IDS];
    int* pos = out + off[F_POSITIONS];
    int* seg = out + off[F_SEG_OF_TOKEN];
    int* seg_start = out + off[F_SEG_START];
    int* seg_pos0 = out + off[F_SEG_POS0];
    int* slot = out + off[F_SLOTS];
    int* rows = out + off[F_LOGIT_ROWS];
    int* tile_seg = out + off[F_TILE_SEG];
    int* tile_q0 = out + off[F_TILE_Q0];
    int* kv_span = out + off[F_KV_SPAN];
    long long kv_sum = 0;
    int kv_longest = 0;
    int cur = 0, row = 0, tile = 0, real = 0, max_kv = cm_info[1];
    const int* tp = tokens;
    const int* wp = want;
    for (int i = 0; i < n; ++i) {
        const int k = n_new[i];
        const bool standin = rids[i] == 0;
        const int p0 = standin ? 0 : starts[real];
        seg_start[i] = cur;
        seg_pos0[i] = p0;
        slot[i] = standin ? scratch[0] : slots[real];
        for (int t = 0; t < k; ++t) {
            tok[cur + t] = tp ? tp[t] : 0;
            pos[cur + t] = p0 + t;
            seg[cur + t] = i;
        }
        if (tp) tp += k;
        for (int w = 0; w < want_n[i]; ++w) rows[row++] = cur + wp[w];
        wp += want_n[i];
        for (int q0 = 0; q0 < k; q0 += query_tile) {
            tile_seg[tile] = i;
            tile_q0[tile] = q0;
            ++tile;
        }
        for (int g = 0; g < groups; ++g) {
            int* bt = out + off[F_BLOCK_TABLE0 + g] + (size_t)i * max_pages;
            if (standin) {
                for (int p = 0; p < max_pages; ++p) bt[p] = scratch[1 + g];
            } else {
                const int* r = gesso_cm_row(cm, rids[i], g, nullptr);
                if (!r) return E_BAD_ARG;
                std::memcpy(bt, r, sizeof(int) * max_pages);
            }
        }
        if (!standin) ++real;
        if (standin && k > max_kv) max_kv = k;
        if (!standin) {                      // stand-ins hold one key on a scratch page: they say nothing about the step
            if (p0 + k > kv_longest) kv_longest = p0 + k;
            kv_sum += p0 + k;
        }
        cur += k;
    }
    seg_start[n] = cur;
    kv_span[0] = kv_longest;
    kv_span[1] = n_real > 0 ? (int)((kv_sum + n_real - 1) / n_real) : 0;
    info[3] = tile;
    for (; tile < cap_tiles; ++tile) {        // the tiles a padded step does not have
        tile_seg[tile] = n - 1;
        tile_q0[tile] = 0;
    }
    info[0] = cm_info[0];
    info[1] = max_kv;
    info[2] = row;
    return OK;
}
