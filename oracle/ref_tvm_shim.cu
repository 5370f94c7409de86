// extern "C" shim around the reference's four fixed-shape TensorFlow-op kernels (Kernels/*.cu: TVM-generated CUDA
// with every shape compiled in), so that the test suite can run them on a GPU and pin the CPU oracle to their outputs.
// TEST INFRASTRUCTURE ONLY.  Built by oracle/build_ref.py into oracle/_ref/, one library per reference file (each
// defines a kernel of the same name), from the reference's sources where they lie, compiled with -DGOOGLE_CUDA=1
// (the files include nothing: no TensorFlow is needed).  Pick the op with -DREF_TVM_<OP>.
//
// Shapes (Kernels/*.cc, test/test_conv2d_rcp.py:17-20, test/test_dense_cp.py:17-20, test/test_conv2d_cp.py:12-23,
// test/test_conv2d_cp4.py:13-25):
//   RCP   U (1,4,4,32,32), K0 (4,4,11), K1 (4,4,11), KC (3,3,11)            -> V (1,4,4,32,32)
//   DENSE U (1,16,16,16), K0, K1, K2 (16,4,137)                              -> V (1,4,4,4)
//   CP3   U (1,16,32,32), K0 (16,6), K1 (3,3,6), K2 (6,16)                   -> V (1,16,32,32)
//   CP4   U (1,16,32,32), K0 (16,6), K1 (3,6), K2 (3,6), K3 (16,6)           -> V (1,16,32,32)
#include <cuda_runtime.h>

#if defined(REF_TVM_RCP)
void Conv2dRcpFusedNchwKernelLauncher(const float* U, const float* K0, const float* K1, const float* KC, float* V);
#define NIN 4
static const size_t kIn[4] = {1 * 4 * 4 * 32 * 32, 4 * 4 * 11, 4 * 4 * 11, 3 * 3 * 11};
static const size_t kOut = 1 * 4 * 4 * 32 * 32;
#define LAUNCH(d, v) Conv2dRcpFusedNchwKernelLauncher(d[0], d[1], d[2], d[3], v)
#elif defined(REF_TVM_DENSE)
void DenseCpKernelLauncher(const float* U, const float* K0, const float* K1, const float* KC, float* V);
#define NIN 4
static const size_t kIn[4] = {16 * 16 * 16, 16 * 4 * 137, 16 * 4 * 137, 16 * 4 * 137};
static const size_t kOut = 4 * 4 * 4;
#define LAUNCH(d, v) DenseCpKernelLauncher(d[0], d[1], d[2], d[3], v)
#elif defined(REF_TVM_CP3)
void Conv2dCpFusedNchwKernelLauncher(const float* U, const float* K0, const float* K1, const float* K2, float* V);
#define NIN 4
static const size_t kIn[4] = {16 * 32 * 32, 16 * 6, 3 * 3 * 6, 6 * 16};
static const size_t kOut = 16 * 32 * 32;
#define LAUNCH(d, v) Conv2dCpFusedNchwKernelLauncher(d[0], d[1], d[2], d[3], v)
#elif defined(REF_TVM_CP4)
void Cp4Conv2dFusedNchwKernelLauncher(const float* U, const float* K0, const float* K1, const float* K2, const float* K3,
                                      float* V);
#define NIN 5
static const size_t kIn[5] = {16 * 32 * 32, 16 * 6, 3 * 6, 3 * 6, 16 * 6};
static const size_t kOut = 16 * 32 * 32;
#define LAUNCH(d, v) Cp4Conv2dFusedNchwKernelLauncher(d[0], d[1], d[2], d[3], d[4], v)
#else
#error "define one of REF_TVM_RCP, REF_TVM_DENSE, REF_TVM_CP3, REF_TVM_CP4"
#endif

// host arrays in, host array out; 0 on success
extern "C" __attribute__((visibility("default"))) int ref_tvm_run(const float* const* in, float* out) {
  float* d[NIN] = {};
  float* v = nullptr;
  int rc = 0;
  for (int i = 0; i < NIN && !rc; ++i) {
    if (cudaMalloc(&d[i], kIn[i] * sizeof(float)) != cudaSuccess) rc = 1;
    else if (cudaMemcpy(d[i], in[i], kIn[i] * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) rc = 1;
  }
  if (!rc && cudaMalloc(&v, kOut * sizeof(float)) != cudaSuccess) rc = 1;
  if (!rc) {
    cudaMemset(v, 0, kOut * sizeof(float));
    LAUNCH(d, v);
    if (cudaDeviceSynchronize() != cudaSuccess) rc = 2;
    else if (cudaMemcpy(out, v, kOut * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) rc = 2;
  }
  for (int i = 0; i < NIN; ++i) cudaFree(d[i]);
  cudaFree(v);
  return rc;
}
