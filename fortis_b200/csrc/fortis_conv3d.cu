// placeholder until the conv3d kernels land
#include "fortis_kernels.h"
#include "fortis_model.h"
namespace fortis {
ConvModel* conv_model_create(const ModelHost&, int, cudaStream_t, std::string* err) { if (err) *err = "conv3d kernel not built"; return nullptr; }
void conv_model_destroy(ConvModel*) {}
bool conv_forward(ConvModel*, const float*, float*, int, int, int, int, cudaStream_t, std::string* err) { if (err) *err = "conv3d kernel not built"; return false; }
bool conv3d_ncdhw(const float*, const float*, float*, int, int, int, int, int, int, int, int, cudaStream_t, std::string* err) { if (err) *err = "conv3d kernel not built"; return false; }
}
