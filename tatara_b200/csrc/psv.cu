// PackedSfenValue records: device-side decode + feature extraction, host-side encoder and the seeded
// synthetic position generator used by the benchmark and the tests.
//
// Record layout (crates/shogi-format/src/packed_sfen.rs:251-271): bytes 0..31 a bit stream read LSB
// first (side to move, two 7-bit king squares, Huffman-coded board, then hand pieces up to bit 256),
// 32..33 score i16 LE, 34..35 move, 36..37 ply u16 LE, 38 result i8, 39 padding.
#include "common.cuh"
#include "../../include/tatara_b200.h"

#include <math.h>
#include <string.h>

#include <vector>

namespace {

// Huffman table, indexed by code id: none, pawn, lance, knight, silver, bishop, rook, gold
// (packed_sfen.rs:26-35); piece types use the reference's numbering (types.rs: pawn 1, lance 2,
// knight 3, silver 4, bishop 5, rook 6, gold 7, king 8, promoted = +8 for pawn..silver, horse 13, dragon 14).
__constant__ unsigned char d_huff_pattern[8] = {0x00, 0x01, 0x03, 0x0b, 0x07, 0x1f, 0x3f, 0x0f};
__constant__ unsigned char d_huff_bits[8] = {1, 2, 4, 4, 4, 6, 6, 5};
const unsigned char h_huff_pattern[8] = {0x00, 0x01, 0x03, 0x0b, 0x07, 0x1f, 0x3f, 0x0f};
const unsigned char h_huff_bits[8] = {1, 2, 4, 4, 4, 6, 6, 5};
// board-piece base of the feature index by piece type: {enemy, friend} (bona_piece.rs:59-90)
__constant__ unsigned short d_piece_base[15][2] = {{0, 0},     {171, 90},   {333, 252},   {495, 414},   {657, 576},
                                                   {981, 900}, {1305, 1224}, {819, 738},   {0, 0},       {819, 738},
                                                   {819, 738}, {819, 738},   {819, 738},   {1143, 1062}, {1467, 1386}};
// hand-piece base by hand slot (pawn, lance, knight, silver, gold, bishop, rook): {enemy, friend}
__constant__ unsigned short d_hand_base[7][2] = {{20, 1}, {44, 39}, {54, 49}, {64, 59}, {74, 69}, {82, 79}, {88, 85}};
// emission order of board pieces (types.rs:271-285)
__constant__ unsigned char d_board_piece_types[13] = {1, 2, 3, 4, 7, 5, 6, 9, 10, 11, 12, 13, 14};

struct FsSpec {
    int kings;   // 0 none, 1 two planes, 2 merged plane
    int mirror;  // king-file mirroring (45 king buckets)
    int piece_inputs;
    int max_active;
};

inline bool fs_spec(int feature_set, FsSpec* s) {
    switch (feature_set) {
        case 0: *s = {0, 0, 1548, 38}; return true;
        case 1: *s = {1, 0, 1710, 40}; return true;
        case 2: *s = {2, 0, 1629, 40}; return true;
        case 3: *s = {1, 1, 1710, 40}; return true;
        case 4: *s = {2, 1, 1629, 40}; return true;
    }
    return false;
}

struct BitReader {
    const unsigned* w;
    int cur;
    __device__ int bit() {
        if (cur >= 256) return 0;
        const int b = (w[cur >> 5] >> (cur & 31)) & 1;
        ++cur;
        return b;
    }
    __device__ unsigned bits(int n) {
        unsigned r = 0;
        for (int i = 0; i < n; ++i) r |= (unsigned)bit() << i;
        return r;
    }
    __device__ unsigned peek(int n) const {
        unsigned r = 0;
        for (int i = 0; i < n; ++i) {
            const int c = cur + i;
            if (c < 256) r |= ((w[c >> 5] >> (c & 31)) & 1u) << i;
        }
        return r;
    }
};

__device__ __forceinline__ int huff_match(unsigned peek, int hand, int* len) {
    for (int i = hand ? 1 : 0; i < 8; ++i) {
        unsigned pattern = d_huff_pattern[i];
        int l = d_huff_bits[i];
        if (hand) { pattern >>= 1; l -= 1; }
        if ((peek & ((1u << l) - 1u)) == pattern) { *len = l; return i; }
    }
    *len = 0;
    return 0;
}

__device__ __forceinline__ int huff_piece_type(int id) {
    // code id -> piece type: pawn, lance, knight, silver, bishop, rook, gold
    const int t[8] = {0, 1, 2, 3, 4, 5, 6, 7};
    return t[id];
}

__device__ __forceinline__ int hand_slot(int pt) {
    // hand order pawn, lance, knight, silver, gold, bishop, rook (types.rs Hand::piece_index)
    switch (pt) {
        case 1: return 0; case 2: return 1; case 3: return 2; case 4: return 3;
        case 7: return 4; case 5: return 5; case 6: return 6;
    }
    return -1;
}

struct Persp {
    int king_bucket;
    int mirror;
    int color;
};

__device__ __forceinline__ Persp make_persp(const FsSpec& s, int king_sq, int color) {
    const int k = color == 0 ? king_sq : 80 - king_sq;
    Persp p;
    p.color = color;
    if (!s.mirror) {
        p.king_bucket = k;
        p.mirror = 0;
    } else {
        const int file = k / 9, rank = k % 9;
        p.king_bucket = (file >= 5 ? 8 - file : file) * 9 + rank;
        p.mirror = file >= 5;
    }
    return p;
}

// feature index of one packed piece value (feature_set.rs:842-845, :972-991)
__device__ __forceinline__ int feat_index(const FsSpec& s, const Persp& p, int bp) {
    if (p.mirror && bp >= 90) {
        const int rel = bp - 90;
        const int piece = rel / 81, sq = rel % 81;
        bp = 90 + piece * 81 + (8 - sq / 9) * 9 + sq % 9;
    }
    if (s.kings == 2 && bp >= 1629) bp -= 81;
    return p.king_bucket * s.piece_inputs + bp;
}

__device__ __forceinline__ int board_bp(int pt, int color, int sq, int persp_color) {
    return d_piece_base[pt][color == persp_color] + (persp_color == 0 ? sq : 80 - sq);
}

// One thread per record.  Emission order: board pieces by (piece type, colour, ascending square), the
// friend and enemy king (when the feature set has king planes), hand pieces of Black then White by
// type and count (feature_set.rs:655-808).  Slots >= nnz are filled with -1.
__global__ void __launch_bounds__(128) k_psv_extract(const unsigned* __restrict__ psv, long long n, FsSpec spec,
                                                      int* __restrict__ stm_out, int* __restrict__ nstm_out,
                                                      int* __restrict__ nnz_out, int* __restrict__ bucket_out,
                                                      float* __restrict__ score_out, float* __restrict__ wdl_out) {
    const long long rec = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (rec >= n) return;
    unsigned w[10];
#pragma unroll
    for (int i = 0; i < 10; ++i) w[i] = psv[rec * 10 + i];
    unsigned char bpt[81], bcol[81];
    unsigned char hand[2][7];
    for (int i = 0; i < 81; ++i) { bpt[i] = 0; bcol[i] = 0; }
    for (int i = 0; i < 14; ++i) hand[i / 7][i % 7] = 0;

    BitReader br{w, 0};
    const int stm = br.bit();
    const int bk = (int)br.bits(7), wk = (int)br.bits(7);
    if (bk < 81) { bpt[bk] = 8; bcol[bk] = 0; }
    if (wk < 81) { bpt[wk] = 8; bcol[wk] = 1; }
    for (int sq = 0; sq < 81; ++sq) {
        if (sq == bk || sq == wk) continue;
        int len;
        const int id = huff_match(br.peek(6), 0, &len);
        br.cur += len;
        if (id == 0) { bpt[sq] = 0; bcol[sq] = 0; continue; }
        const int promoted = id != 7 ? br.bit() : 0;
        const int color = br.bit();
        int pt = huff_piece_type(id);
        if (promoted) pt = pt <= 4 ? pt + 8 : (pt == 5 ? 13 : 14);
        bpt[sq] = (unsigned char)pt;
        bcol[sq] = (unsigned char)color;
    }
    while (br.cur < 256) {
        int len;
        const int id = huff_match(br.peek(5), 1, &len);
        br.cur += len;
        const int piecebox = id != 7 ? br.bit() : 0;
        const int color = br.bit();
        if (piecebox) continue;  // piece-box entries (handicap games) are not hand pieces
        const int slot = hand_slot(huff_piece_type(id));
        if (slot >= 0) hand[color][slot]++;
    }

    const int A = spec.max_active;
    int* so = stm_out + rec * A;
    int* no = nstm_out + rec * A;
    int count = 0;
    const int nstm = stm ^ 1;
    const int stm_king = stm == 0 ? bk : wk, nstm_king = nstm == 0 ? bk : wk;
    if (stm_king < 81 && nstm_king < 81) {
        const Persp sp = make_persp(spec, stm_king, stm), np = make_persp(spec, nstm_king, nstm);
        // counting pass: slot base of every (piece type, colour) group in emission order
        unsigned char cnt[30];
        for (int i = 0; i < 30; ++i) cnt[i] = 0;
        for (int sq = 0; sq < 81; ++sq) {
            const int pt = bpt[sq];
            if (pt != 0 && pt != 8) cnt[pt * 2 + bcol[sq]]++;
        }
        unsigned char base[30];
        int run = 0;
        for (int t = 0; t < 13; ++t)
            for (int c = 0; c < 2; ++c) {
                const int g = d_board_piece_types[t] * 2 + c;
                base[g] = (unsigned char)run;
                run += cnt[g];
            }
        for (int sq = 0; sq < 81; ++sq) {
            const int pt = bpt[sq];
            if (pt == 0 || pt == 8) continue;
            const int c = bcol[sq];
            const int slot = base[pt * 2 + c]++;
            if (slot < A) {
                so[slot] = feat_index(spec, sp, board_bp(pt, c, sq, stm));
                no[slot] = feat_index(spec, np, board_bp(pt, c, sq, nstm));
            }
        }
        count = run < A ? run : A;
        if (spec.kings != 0) {
            if (count < A) {
                so[count] = feat_index(spec, sp, 1548 + (stm == 0 ? stm_king : 80 - stm_king));
                no[count] = feat_index(spec, np, 1548 + (nstm == 0 ? nstm_king : 80 - nstm_king));
                ++count;
            }
            if (count < A) {
                so[count] = feat_index(spec, sp, 1629 + (stm == 0 ? nstm_king : 80 - nstm_king));
                no[count] = feat_index(spec, np, 1629 + (nstm == 0 ? stm_king : 80 - stm_king));
                ++count;
            }
        }
        for (int owner = 0; owner < 2; ++owner)
            for (int slot = 0; slot < 7; ++slot) {
                const int nh = hand[owner][slot];
                for (int i = 1; i <= nh; ++i) {
                    if (count >= A) break;
                    so[count] = feat_index(spec, sp, d_hand_base[slot][owner == stm] + i - 1);
                    no[count] = feat_index(spec, np, d_hand_base[slot][owner == nstm] + i - 1);
                    ++count;
                }
            }
    }
    for (int k = count; k < A; ++k) { so[k] = -1; no[k] = -1; }
    nnz_out[rec] = count;
    const short score = (short)(w[8] & 0xffffu);
    const signed char result = (signed char)((w[9] >> 16) & 0xffu);
    score_out[rec] = (float)score;
    wdl_out[rec] = result > 0 ? 1.0f : (result < 0 ? 0.0f : 0.5f);
    if (bucket_out) {
        // kingrank9 (crates/shogi-features/src/kingrank9.rs:11-24)
        const int friendly = stm == 0 ? bk : 80 - wk;
        const int enemy = stm == 0 ? 80 - wk : bk;
        bucket_out[rec] = ((friendly % 9) / 3) * 3 + (enemy % 9) / 3;
    }
}

struct BitWriter {
    uint8_t* data;
    int cur;
    void put(unsigned v, int n) {
        for (int i = 0; i < n; ++i, ++cur)
            if ((v >> i) & 1u) data[cur >> 3] |= (uint8_t)(1u << (cur & 7));
    }
};

int huff_id_of(int base_pt) {
    switch (base_pt) {
        case 1: return 1; case 2: return 2; case 3: return 3; case 4: return 4;
        case 5: return 5; case 6: return 6; case 7: return 7;
    }
    return 0;
}

struct SplitMix64 {
    uint64_t s;
    uint64_t next() {
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double unit() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
    uint32_t below(uint32_t n) { return (uint32_t)(((next() >> 32) * (uint64_t)n) >> 32); }
};

}  // namespace

extern "C" int tb_psv_encode(const uint8_t* board_pt, const uint8_t* board_color, const uint8_t* hand_black7,
                             const uint8_t* hand_white7, int side_to_move, int black_king_sq, int white_king_sq,
                             int score, int ply, int result, uint8_t* out) {
    if (!board_pt || !board_color || !hand_black7 || !hand_white7 || !out) return TB_ERR_INVALID_ARGUMENT;
    memset(out, 0, 40);
    BitWriter bw{out, 0};
    bw.put((unsigned)side_to_move & 1u, 1);
    bw.put((unsigned)black_king_sq, 7);
    bw.put((unsigned)white_king_sq, 7);
    for (int sq = 0; sq < 81; ++sq) {
        if (sq == black_king_sq || sq == white_king_sq) continue;
        int pt = board_pt[sq];
        if (pt == 0) { bw.put(0, 1); continue; }
        int promoted = 0, base = pt;
        if (pt >= 9 && pt <= 12) { promoted = 1; base = pt - 8; }
        else if (pt == 13) { promoted = 1; base = 5; }
        else if (pt == 14) { promoted = 1; base = 6; }
        const int id = huff_id_of(base);
        if (id == 0) return TB_ERR_INVALID_ARGUMENT;
        bw.put(h_huff_pattern[id], h_huff_bits[id]);
        if (id != 7) bw.put((unsigned)promoted, 1);
        bw.put(board_color[sq] & 1u, 1);
        if (bw.cur > 256) return TB_ERR_INVALID_ARGUMENT;
    }
    // hand pieces: code without its first bit, a piece-box flag of 0 (not for gold), colour
    static const int slot_pt[7] = {1, 2, 3, 4, 7, 5, 6};
    for (int color = 0; color < 2; ++color) {
        const uint8_t* h = color == 0 ? hand_black7 : hand_white7;
        for (int slot = 0; slot < 7; ++slot)
            for (int k = 0; k < h[slot]; ++k) {
                const int id = huff_id_of(slot_pt[slot]);
                bw.put((unsigned)h_huff_pattern[id] >> 1, h_huff_bits[id] - 1);
                if (id != 7) bw.put(0, 1);
                bw.put((unsigned)color, 1);
                if (bw.cur > 256) return TB_ERR_INVALID_ARGUMENT;
            }
    }
    const int16_t sc = (int16_t)score;
    out[32] = (uint8_t)(sc & 0xff);
    out[33] = (uint8_t)((sc >> 8) & 0xff);
    out[36] = (uint8_t)(ply & 0xff);
    out[37] = (uint8_t)((ply >> 8) & 0xff);
    out[38] = (uint8_t)(int8_t)result;
    return TB_OK;
}

// Synthetic positions.  Every record holds the full 40-piece set, which always fills the 256 bits
// exactly.  Drawn from one SplitMix64 stream in this order per record: side to move (1 bit), black
// king square (uniform of 81), white king square (uniform of the other 80); then for each of the 38
// other pieces in the order 18 pawns, 4 lances, 4 knights, 4 silvers, 4 golds, 2 bishops, 2 rooks:
// on the board with p = 0.85 (uniform empty square, uniform owner, promoted with p = 0.1 unless gold),
// otherwise in the hand of a uniform side; score = round(400 * N(0,1)) clipped to +-3000 (Box-Muller);
// result = draw with p = 0.05, else win with p = sigmoid(score / 600), else loss; ply uniform in 1..256.
// Legality of the position is not enforced (the extractor does not need it).
extern "C" int tb_psv_synthesize(uint64_t seed, int64_t n_records, uint8_t* out) {
    if (n_records < 0 || (n_records > 0 && !out)) return TB_ERR_INVALID_ARGUMENT;
    SplitMix64 rng{seed};
    static const int piece_list[7][2] = {{1, 18}, {2, 4}, {3, 4}, {4, 4}, {7, 4}, {5, 2}, {6, 2}};
    for (int64_t r = 0; r < n_records; ++r) {
        uint8_t pt[81] = {0}, col[81] = {0}, hand[2][7] = {{0}};
        const int stm = (int)(rng.next() & 1u);
        const int bk = (int)rng.below(81);
        int wk = (int)rng.below(80);
        if (wk >= bk) ++wk;
        pt[bk] = 8; col[bk] = 0;
        pt[wk] = 8; col[wk] = 1;
        int empties = 79;
        for (int t = 0; t < 7; ++t)
            for (int k = 0; k < piece_list[t][1]; ++k) {
                const int type = piece_list[t][0];
                if (rng.unit() < 0.85) {
                    int pick = (int)rng.below((uint32_t)empties), sq = 0;
                    for (;; ++sq)
                        if (pt[sq] == 0 && pick-- == 0) break;
                    const int owner = (int)(rng.next() & 1u);
                    int placed = type;
                    if (type != 7 && rng.unit() < 0.1) placed = type <= 4 ? type + 8 : (type == 5 ? 13 : 14);
                    pt[sq] = (uint8_t)placed;
                    col[sq] = (uint8_t)owner;
                    --empties;
                } else {
                    const int owner = (int)(rng.next() & 1u);
                    static const int slot_of[8] = {-1, 0, 1, 2, 3, 5, 6, 4};
                    hand[owner][slot_of[type]]++;
                }
            }
        double u1 = rng.unit();
        if (u1 < 1e-300) u1 = 1e-300;
        const double u2 = rng.unit();
        const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
        long sc = lrint(z * 400.0);
        if (sc > 3000) sc = 3000;
        if (sc < -3000) sc = -3000;
        int result;
        if (rng.unit() < 0.05) result = 0;
        else result = rng.unit() < 1.0 / (1.0 + exp(-(double)sc / 600.0)) ? 1 : -1;
        const int ply = 1 + (int)rng.below(256);
        const int rc = tb_psv_encode(pt, col, hand[0], hand[1], stm, bk, wk, (int)sc, ply, result, out + 40 * r);
        if (rc != TB_OK) return rc;
    }
    return TB_OK;
}

// Device-to-device form for the trainer: records already in device memory -> step inputs in device memory, on `s`.
// Returns the number of kernels launched, or -1 for an unknown feature set.
int launch_psv_extract(cudaStream_t s, int feature_set, const void* d_psv, long long n, int* stm, int* nstm, int* nnz,
                       int* bucket, float* score, float* wdl) {
    FsSpec spec;
    if (!fs_spec(feature_set, &spec)) return -1;
    if (n <= 0) return 0;
    k_psv_extract<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(static_cast<const unsigned*>(d_psv), n, spec, stm, nstm, nnz, bucket, score, wdl);
    return 1;
}

// dimensions of a feature set id: rows of the FT table and slots per perspective (feature_set.rs:1031-1038)
bool psv_feature_set_dims(int feature_set, int* ft_in, int* max_active) {
    FsSpec spec;
    if (!fs_spec(feature_set, &spec)) return false;
    *ft_in = (spec.mirror ? 45 : 81) * spec.piece_inputs;
    *max_active = spec.max_active;
    return true;
}

extern "C" int tb_psv_extract(int device, int feature_set, const uint8_t* psv, int64_t n, int32_t* stm_indices,
                              int32_t* nstm_indices, int32_t* nnz, int32_t* bucket, float* score, float* wdl) {
    FsSpec spec;
    if (!fs_spec(feature_set, &spec) || n < 0) return TB_ERR_INVALID_ARGUMENT;
    if (n == 0) return TB_OK;
    if (!psv || !stm_indices || !nstm_indices || !nnz || !score || !wdl) return TB_ERR_INVALID_ARGUMENT;
    if (cudaSetDevice(device) != cudaSuccess) return TB_ERR_NO_DEVICE;
    const size_t A = (size_t)spec.max_active;
    unsigned* d_psv = nullptr;
    int *d_stm = nullptr, *d_nstm = nullptr, *d_nnz = nullptr, *d_bucket = nullptr;
    float *d_score = nullptr, *d_wdl = nullptr;
    cudaError_t e = cudaSuccess;
    auto chk = [&](cudaError_t x) { if (e == cudaSuccess) e = x; };
    chk(cudaMalloc(&d_psv, (size_t)n * 40));
    chk(cudaMalloc(&d_stm, (size_t)n * A * 4));
    chk(cudaMalloc(&d_nstm, (size_t)n * A * 4));
    chk(cudaMalloc(&d_nnz, (size_t)n * 4));
    chk(cudaMalloc(&d_bucket, (size_t)n * 4));
    chk(cudaMalloc(&d_score, (size_t)n * 4));
    chk(cudaMalloc(&d_wdl, (size_t)n * 4));
    if (e == cudaSuccess) {
        chk(cudaMemcpy(d_psv, psv, (size_t)n * 40, cudaMemcpyHostToDevice));
        k_psv_extract<<<(unsigned)((n + 127) / 128), 128>>>(d_psv, n, spec, d_stm, d_nstm, d_nnz, d_bucket, d_score, d_wdl);
        chk(cudaGetLastError());
        chk(cudaMemcpy(stm_indices, d_stm, (size_t)n * A * 4, cudaMemcpyDeviceToHost));
        chk(cudaMemcpy(nstm_indices, d_nstm, (size_t)n * A * 4, cudaMemcpyDeviceToHost));
        chk(cudaMemcpy(nnz, d_nnz, (size_t)n * 4, cudaMemcpyDeviceToHost));
        if (bucket) chk(cudaMemcpy(bucket, d_bucket, (size_t)n * 4, cudaMemcpyDeviceToHost));
        chk(cudaMemcpy(score, d_score, (size_t)n * 4, cudaMemcpyDeviceToHost));
        chk(cudaMemcpy(wdl, d_wdl, (size_t)n * 4, cudaMemcpyDeviceToHost));
    }
    cudaFree(d_psv); cudaFree(d_stm); cudaFree(d_nstm); cudaFree(d_nnz); cudaFree(d_bucket); cudaFree(d_score); cudaFree(d_wdl);
    return e == cudaSuccess ? TB_OK : TB_ERR_CUDA;
}
