// C API of the fused optimizer kernels (sm_100a). One call updates one contiguous tensor in place.
// dtype codes: 0 = fp32, 1 = fp16, 2 = bf16 (parameter and gradient share the dtype).
// Moment state is fp32 (adamw, muon) or uint8 codes + one fp32 absmax per 256 values (8-bit variants);
// `lut` is the 256-entry dynamic code book (device pointer) or NULL for the symmetric int8 codec.
// Counterpart of cppmega_mlx/training/native_optim/fused_8bit.h:19-48 in the reference.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int cmb_adamw(void* p, const void* g, float* m, float* v, int64_t n, int dtype, float lr, float b1, float b2, float eps,
              float wd, float c1, float c2, float grad_scale, void* stream);
int cmb_adam8bit(void* p, const void* g, uint8_t* mq, float* ma, uint8_t* vq, float* va, const float* lut, int64_t n,
                 int dtype, float lr, float b1, float b2, float eps, float wd, float c1, float c2, void* stream);
int cmb_lion8bit(void* p, const void* g, uint8_t* mq, float* ma, const float* lut, int64_t n, int dtype, float lr,
                 float b1, float b2, float wd, void* stream);
int cmb_muon_momentum(const void* g, const void* p, float* v, void* out_bf16, float* sumsq, int64_t n, int dtype,
                      float momentum, float wd, int nesterov, void* stream);
int cmb_scale_inv_norm(void* x_bf16, const float* sumsq, int64_t n, float eps, void* stream);
int cmb_axpy_update(void* p, const void* u_bf16, int64_t n, int dtype, float coef, void* stream);
#ifdef __cplusplus
}
#endif
