/*
 * TEST INFRASTRUCTURE -- CPU oracle for libd2conv3d.
 *
 * A plain-C restatement of the reference's algorithm for the deformable /
 * dynamic-dilated / depthwise conv3d path (Schmiddo/d2conv3d:
 * ops/dconv-native/csrc/ops/dconv3d_gpu.cu, utils/grid.py,
 * ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu).  The reference has no CPU
 * implementation of this path (every tensor must be CUDA), so this file is the
 * checker the GPU kernels are compared with.  It is pinned against the
 * reference's own executable test oracle (`expected_fn`,
 * ops/dconv-native/test/test_deform_conv.py:127-191), its conv3d identities and
 * its offsets_from_size_map through the fixtures in tests/golden/.
 *
 * Only tests, the smoke check and the bench's CPU-baseline legs may load this
 * library; the product never does.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/d2conv3d.h"

typedef struct orc_geom {
  int B, Cin, Cout, D, H, W, kd, kh, kw, sd, sh, sw, pd, ph, pw, dd, dh, dw, groups, G;
  int Do, Ho, Wo, K, V;
} orc_geom;

/* get_output_size, ops/dconv-native/csrc/ops/dconv_gpu_common.h:13-15 */
static int orc_out_size(int in, int k, int s, int p, int d) { return (in + 2 * p - (d * (k - 1) + 1)) / s + 1; }

static int orc_fill(const d2c_conv_desc* d, orc_geom* g) {
  g->B = d->batch; g->Cin = d->in_channels; g->Cout = d->out_channels;
  g->D = d->in_d; g->H = d->in_h; g->W = d->in_w;
  g->kd = d->kd; g->kh = d->kh; g->kw = d->kw;
  g->sd = d->stride_d; g->sh = d->stride_h; g->sw = d->stride_w;
  g->pd = d->pad_d; g->ph = d->pad_h; g->pw = d->pad_w;
  g->dd = d->dil_d; g->dh = d->dil_h; g->dw = d->dil_w;
  g->groups = d->groups; g->G = d->offset_groups;
  if (g->kd <= 0 || g->kh <= 0 || g->kw <= 0 || g->sd <= 0 || g->sh <= 0 || g->sw <= 0 ||
      g->dd <= 0 || g->dh <= 0 || g->dw <= 0 || g->pd < 0 || g->ph < 0 || g->pw < 0)
    return -1;
  if (g->kd > 64 || g->kh > 64 || g->kw > 64) return -1;
  g->Do = orc_out_size(g->D, g->kd, g->sd, g->pd, g->dd);
  g->Ho = orc_out_size(g->H, g->kh, g->sh, g->ph, g->dh);
  g->Wo = orc_out_size(g->W, g->kw, g->sw, g->pw, g->dw);
  if (g->Do <= 0 || g->Ho <= 0 || g->Wo <= 0) return -1;
  g->K = g->kd * g->kh * g->kw;
  g->V = g->Do * g->Ho * g->Wo;
  return 0;
}

/* group rules of SANITY_CHECK_DCONV_GROUPS, dconv_gpu_common.h:19-25 */
static int orc_make_geom(const d2c_conv_desc* d, orc_geom* g) {
  if (orc_fill(d, g)) return -1;
  if (g->groups <= 0 || g->G <= 0) return -1;
  if (g->Cin % g->groups || g->Cout % g->groups || g->Cout % g->G || g->Cin % g->G) return -1;
  return 0;
}

/* depthwise rule of conv_depthwise_shape_check, grouped_conv3d.cu:303-308 */
static int orc_make_geom_dw(const d2c_conv_desc* d, orc_geom* g) {
  if (orc_fill(d, g)) return -1;
  if (g->Cin <= 0 || g->Cout % g->Cin) return -1;
  return 0;
}

/* OpenMP team size of the loops below.  A launcher may have exported OMP_NUM_THREADS=1 before this library was
 * loaded (torchrun does for every rank); the timing legs set the team size explicitly instead. */
#ifdef _OPENMP
#include <omp.h>
int orc_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}
#else
int orc_set_threads(int n) { (void)n; return 1; }
#endif

int orc_output_dims(const d2c_conv_desc* d, int32_t out[3]) {
  orc_geom g;
  if (orc_fill(d, &g)) return -1;
  out[0] = g.Do; out[1] = g.Ho; out[2] = g.Wo;
  return 0;
}

/* which size_map channel feeds dim d (0:z 1:y 2:x); -1 = constant one.
 * utils/grid.py:79-92. */
static int orc_field_channel(int mode, int d) {
  switch (mode) {
    case D2C_FIELD_X: return d == 0 ? -1 : 0;
    case D2C_FIELD_XY: return d == 0 ? -1 : d - 1;
    case D2C_FIELD_XXZ: return d == 0 ? 0 : 1;
    default: return d;
  }
}
static int orc_field_channels(int mode) {
  return mode == D2C_FIELD_X ? 1 : (mode == D2C_FIELD_XYZ ? 3 : 2);
}

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define T float
#define FN(name) CAT(name, _f32)
#define FLOOR floorf
#define FABS fabsf
#define FMA fmaf
#include "d2c_oracle_impl.inc"
#undef T
#undef FN
#undef FLOOR
#undef FABS
#undef FMA

#define T double
#define FN(name) CAT(name, _f64)
#define FLOOR floor
#define FABS fabs
#define FMA fma
#include "d2c_oracle_impl.inc"
#undef T
#undef FN
#undef FLOOR
#undef FABS
#undef FMA
