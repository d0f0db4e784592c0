#include "deform_sm100.h"

namespace d2c {

bool sm100_fwd_supported(const Geom&, int, int) { return false; }
size_t sm100_fwd_workspace(const Geom&, int, int) { return 0; }
size_t sm100_bwd_workspace(const Geom&, int, int) { return 0; }
int sm100_fwd_offsets(const Geom&, int, const float*, const float*, const float*, const float*,
                      const float*, float*, void*, cudaStream_t) { return D2C_ERR_MODE; }
int sm100_fwd_field(const Geom&, int, const FieldCoords<float>&, const float*, const float*,
                    const float*, const float*, float*, void*, cudaStream_t) { return D2C_ERR_MODE; }

}  // namespace d2c
