// Host-side (pure CPU) load-time helpers: the escape table and non-empty row
// list the engine builds after reading a tensor (engine/model.cpp:86-156 of the
// reference), and tensor-parallel sharding of a packed tensor, which the
// single-GPU reference does not have.
#include <cstdint>
#include <cstring>
#include <vector>
#include "../../include/split12_b200.h"

extern "C" {

int s12_host_build_escape_table(const int32_t* row_off, const int32_t* cols,
                                const int16_t* correct, int M,
                                int32_t* row_base, uint8_t* counts, int16_t* vals,
                                int32_t* nonempty_rows)
{
    if (M < 0 || (M > 0 && (!row_off || !row_base))) return S12_ERR_BAD_ARG;
    int nne = 0;
    std::vector<int32_t> slot(256);
    for (int r = 0; r < M; r++) {
        const int32_t lo = row_off[r], hi = row_off[r + 1];
        row_base[r] = lo;
        if (counts) std::memset(counts + (size_t)r * 256, 0, 256);
        if (hi <= lo) continue;
        if (!cols || !correct || !vals) return S12_ERR_BAD_ARG;
        if (nonempty_rows) nonempty_rows[nne] = r;
        nne++;
        // counting sort of the row's escapes by (col mod 256); stable, so equal
        // residues keep ascending column order
        std::fill(slot.begin(), slot.end(), 0);
        for (int32_t p = lo; p < hi; p++) slot[cols[p] & 255]++;
        int32_t run = lo;
        for (int t = 0; t < 256; t++) {
            int32_t n = slot[t];
            if (counts) counts[(size_t)r * 256 + t] = (uint8_t)n;
            slot[t] = run;
            run += n;
        }
        for (int32_t p = lo; p < hi; p++) vals[slot[cols[p] & 255]++] = correct[p];
    }
    return nne;
}

int64_t s12_host_shard_rows(const S12Tensor* src, int r0, int r1,
                            uint8_t* sm, uint8_t* gr, int32_t* row_off,
                            int32_t* cols, int16_t* correct, int16_t* wrong)
{
    if (!src || !sm || !gr || !row_off) return S12_ERR_BAD_ARG;
    const int64_t K = src->K;
    if (r0 < 0 || r1 < r0 || r1 > src->M || (K & 1)) return S12_ERR_BAD_ARG;
    const int64_t rows = r1 - r0;
    std::memcpy(sm, src->sm + (int64_t)r0 * K, (size_t)(rows * K));
    std::memcpy(gr, src->gr + ((int64_t)r0 * K) / 2, (size_t)(rows * K / 2));
    if (!src->row_off) {
        for (int64_t r = 0; r <= rows; r++) row_off[r] = 0;
        return 0;
    }
    const int32_t first = src->row_off[r0];
    const int64_t n = src->row_off[r1] - first;
    for (int64_t r = 0; r <= rows; r++) row_off[r] = src->row_off[r0 + r] - first;
    if (n > 0) {
        if (!cols || !correct || !wrong) return S12_ERR_BAD_ARG;
        std::memcpy(cols, src->cols + first, (size_t)n * sizeof(int32_t));
        std::memcpy(correct, src->correct + first, (size_t)n * sizeof(int16_t));
        std::memcpy(wrong, src->wrong + first, (size_t)n * sizeof(int16_t));
    }
    return n;
}

int64_t s12_host_shard_cols(const S12Tensor* src, int c0, int c1,
                            uint8_t* sm, uint8_t* gr, int32_t* row_off,
                            int32_t* cols, int16_t* correct, int16_t* wrong)
{
    if (!src || !sm || !gr || !row_off) return S12_ERR_BAD_ARG;
    const int64_t K = src->K, M = src->M;
    // nibble pairs must not be split: even cuts of an even K
    if (c0 < 0 || c1 < c0 || c1 > K || (c0 & 1) || (c1 & 1) || (K & 1)) return S12_ERR_BAD_ARG;
    const int64_t Ks = c1 - c0;
    int64_t n = 0;
    row_off[0] = 0;
    for (int64_t r = 0; r < M; r++) {
        std::memcpy(sm + r * Ks, src->sm + r * K + c0, (size_t)Ks);
        std::memcpy(gr + (r * Ks) / 2, src->gr + (r * K + c0) / 2, (size_t)(Ks / 2));
        if (src->row_off) {
            for (int32_t p = src->row_off[r]; p < src->row_off[r + 1]; p++) {
                const int32_t c = src->cols[p];
                if (c < c0 || c >= c1) continue;
                if (!cols || !correct || !wrong) return S12_ERR_BAD_ARG;
                cols[n] = c - c0; correct[n] = src->correct[p]; wrong[n] = src->wrong[p];
                n++;
            }
        }
        row_off[r + 1] = (int32_t)n;
    }
    return n;
}

}  // extern "C"
