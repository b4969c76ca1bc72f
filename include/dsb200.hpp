// C++ convenience layer over dsb200.h for callers of the reference's torch-free C++ API
// ("Native CPP (Thrust) and Torch I/O API", cpp/ds_cuda_rasterizer/rasterizer_cuda.hpp:4-9).
#ifndef DSB200_HPP_
#define DSB200_HPP_
#include <stdexcept>
#include <string>

#include "dsb200.h"

namespace dsb200 {

// Drop-in for the reference's function of the same name: device pointers in, device image [H][W][3] out, on the
// given stream (the reference uses the default stream).  Throws std::runtime_error where the reference would have
// failed a CUDA call silently.
inline void rasterizer_forward_core_deepsense(const float* means_3d, const float* shs, const float* opacities,
                                              const float* scales, const float* rotations, int num_of_gaussians,
                                              const float* view_matrix, const float* proj_matrix,
                                              const float* camera_position, int image_width, int image_height,
                                              float tan_fovx, float tan_fovy, float scale_modifier,
                                              const int max_sh_degree, const int sh_degree, float* output_image,
                                              void* stream = nullptr) {
    const int rc = dsb_forward_core(means_3d, shs, opacities, scales, rotations, num_of_gaussians, view_matrix, proj_matrix,
                                    camera_position, image_width, image_height, tan_fovx, tan_fovy, scale_modifier,
                                    max_sh_degree, sh_degree, output_image, stream);
    if (rc != DSB_OK) throw std::runtime_error(std::string("dsb200: ") + dsb_last_error());
}

}  // namespace dsb200
#endif  // DSB200_HPP_
