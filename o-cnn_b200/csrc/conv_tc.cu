// Placeholder translation unit for the tensor-core convolution (filled in by conv_tc.cu proper).
#include "common.cuh"

extern "C" {

size_t ocnn_conv_packed_weight_bytes(int cin, int cout, const int kernel_size[3]) {
  (void)cin; (void)cout; (void)kernel_size;
  return 0;
}

int ocnn_conv_pack_weights(const float*, void*, int, int, const int*, void*) {
  return ocnn::fail(OCNN_ERR_UNSUPPORTED, "tensor-core convolution not built");
}

int ocnn_octree_conv_tc(const void*, const void*, void*, const int32_t*, int, int, int, int,
                        const int*, int, const ocnn_conv_epilogue*, int32_t*, void*) {
  return ocnn::fail(OCNN_ERR_UNSUPPORTED, "tensor-core convolution not built");
}

}
