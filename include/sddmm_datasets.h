/*
 * sddmm_datasets.h -- seeded synthetic SDDMM inputs (host only, no CUDA).
 *
 * The matrices francois141/dphpc measures on come from SuiteSparse/SNAP
 * (install_matrices.sh) and its random inputs are unseeded
 * (src/utils/random_generator.hpp:13-14).  These generators stand in for them
 * with fixed seeds so that every run, every rank and every language binding
 * sees bit-identical inputs.  Shapes follow README.md:22,36,53,55,56 of that
 * project (ex21, human_gene2, inline_1, sx-stackoverflow, nv2).
 *
 *   config 1  small uniform      656 x 656,        18 964 nnz
 *   config 2  clustered blocks   14 340 x 14 340,  ~18.07 M nnz (64x64 blocks, 70 % full)
 *   config 3  banded 3x3 blocks  503 712 x 503 712, ~36.8 M nnz, half-width 2000
 *   config 4  power law          2 601 977^2,      ~36.2 M nnz, Zipf(2) rows and columns
 *   config 5  Poisson rows       1 453 908^2,      ~37.5 M nnz, uniform columns
 *
 * `scale` in (0, 1] shrinks the number of rows/columns (per-row statistics are
 * kept) so that the same structure can be checked against a CPU oracle quickly.
 * Output: CSR with sorted, duplicate-free columns in every row -- the arrays the
 * reference's CSR<T>(rows, cols, triplets) constructor (src/matrices/CSR.hpp:29-32,
 * 169-194) produces from the same triplets -- plus A (M x K) and B (N x K),
 * row-major fp32 in [-1, 1); S values in [0, 1) (all 1.0 for config 4).
 */
#ifndef SDDMM_DATASETS_H
#define SDDMM_DATASETS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sddmm_dataset sddmm_dataset;

/* config in 1..5; K >= 1; 0 < scale <= 1; variant: 0 = default; config 2 only: 1 = unaligned block origins */
int sddmm_dataset_create(sddmm_dataset **out, int config, int64_t K, double scale, uint64_t seed, int variant);
/* uniformly random pattern with exactly nnz distinct positions (the analogue of
 * RandomWithDensityDataset, src/benchmark/dataset.hpp:331-356) */
int sddmm_dataset_create_uniform(sddmm_dataset **out, int64_t M, int64_t N, int64_t K, int64_t nnz, uint64_t seed);
void sddmm_dataset_destroy(sddmm_dataset *ds);

void sddmm_dataset_dims(const sddmm_dataset *ds, int64_t *M, int64_t *N, int64_t *K, int64_t *nnz);
const char *sddmm_dataset_name(const sddmm_dataset *ds);
const int32_t *sddmm_dataset_row_ptr(const sddmm_dataset *ds);
const int32_t *sddmm_dataset_col_idx(const sddmm_dataset *ds);
const float *sddmm_dataset_s_val(const sddmm_dataset *ds);
const float *sddmm_dataset_A(const sddmm_dataset *ds);
const float *sddmm_dataset_B(const sddmm_dataset *ds);

#ifdef __cplusplus
}
#endif
#endif
