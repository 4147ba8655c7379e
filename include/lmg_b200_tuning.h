/* Tuning knobs and measurement hooks of liblmg_b200.so.  None of these has a counterpart in the
 * reference: they select between kernels that give the same results, or expose counters that
 * bench.py reads.  All settings are process-wide and meant to be changed between calls only. */
#ifndef LMG_B200_TUNING_H_
#define LMG_B200_TUNING_H_
#ifdef __cplusplus
extern "C" {
#endif

/* -1 (default): the reference's own operation order for the density when gaussian_radius_multiple > 2,
 * the fast form otherwise; 0 / 1 force the fast / exact form. */
void lmg_set_precise(int mode);
/* 1 (default): kernels that walk rows in aligned quads of four voxels (16-byte loads,
 * red.global.add.v4.f32) where dim % 4 == 0 and the grid is 16-byte aligned; 0: never. */
void lmg_set_quads(int on);
/* 1 (default): GridInterpolater stages input boxes through tensor copies where rows of the input
 * are 16-byte aligned and out_resolution <= in_resolution; 0: always the direct-read kernel. */
void lmg_set_interp_tiled(int on);
/* Blocks of the tiled interpolation kernel that ever gave up a bounded wait for a staged box (they
 * finish through direct reads, so results stay correct); 0xffffffff if the counter cannot be read. */
unsigned lmg_tma_timeouts(void);

/* Per-kernel CUDA-event timing: enable with the number of records to keep (0 disables), then
 * collect sums of milliseconds and counts per kind {0 forward kernels, 1 backward kernels, 2 zero
 * fill}; collecting synchronises the recorded events. */
int lmg_profile_enable(int max_records);
int lmg_profile_collect(double ms[3], int count[3]);
/* Kernels this library has launched in this process. */
long lmg_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* LMG_B200_TUNING_H_ */
