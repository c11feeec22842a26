/* mam_b200_tuning.h -- test and tuning hooks of libmam_b200.so.
 *
 * NOT part of the drop-in boundary (include/mam_b200.h): nothing here has a counterpart in
 * SSIGPRO/mamtorch and no caller of the library needs it.  The parity tests use these knobs to run
 * every kernel form against the oracle, and timing sweeps use them to compare forms.  All knobs
 * are process-wide and not thread-safe; every one defaults to "chosen by shape".
 */
#ifndef MAM_B200_TUNING_H
#define MAM_B200_TUNING_H

#ifdef __cplusplus
extern "C" {
#endif

enum mam_tune_knob {
    MAM_TUNE_FWD_VALUES = 0,   /* tile configuration of the values-only tiled forward: -1 by shape, -2 the
                                  any-shape kernel, 0.. index mam_fwd_variant_name(0, i)                     */
    MAM_TUNE_FWD_INDICES = 1,  /* the same for the index-producing forward, names from mam_fwd_variant_name(1, i) */
    MAM_TUNE_RESOLVER = 2,     /* 0 tiled index resolver (default), 1 one thread per output                   */
    MAM_TUNE_BWD_FORM = 3,     /* 0 by shape, 1 CTA-shared rows of dX, 2 separate dX and dW kernels,
                                  3 / 4 one row of dX per warp (a parked in shared memory / read through L1)  */
    MAM_TUNE_DENSE_SPLIT = 4,  /* TF32 product: 1 slices the tiles of the last partial wave (default), 0 not  */
    MAM_TUNE_CONV_DIRECT_ROWS = 5 /* output rows per CTA of the one-kernel convolution backward, 0 by size    */
};

/* Sets one knob; MAM_ERR_INVALID_ARGUMENT for an unknown knob or a value outside its range. */
int mam_tune_set(int knob, int value);
/* Name of tile configuration `variant` of the values-only (with_indices = 0) or index-producing
 * (1) forward; "auto" for -1, "generic" for -2, "" outside the table. */
const char* mam_fwd_variant_name(int with_indices, int variant);

#ifdef __cplusplus
}
#endif
#endif /* MAM_B200_TUNING_H */
