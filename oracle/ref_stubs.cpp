// Link-time stand-ins for the reference's per-WxAy GPU benchmark drivers (engine/test/test_mma/*.cu),
// which engine/test_any_mma.cu calls from its main().  The oracle library only uses the host
// functions of that file (compute_ref, init_matrix, int_pow) and the pack launchers, so the drivers
// are never called; these definitions exist only so the shared object has no unresolved symbols.
#include <cuda_runtime.h>
#define ABQ_REF_STUB(name)                                                                          \
    void name(int, int, int *, int *, int *, int *, int, int, int, int *, int *, int *, int, int,  \
              bool, cudaStream_t)                                                                   \
    {                                                                                               \
    }
ABQ_REF_STUB(test_mma_w2a2)
ABQ_REF_STUB(test_mma_w2a4)
ABQ_REF_STUB(test_mma_w2a6)
ABQ_REF_STUB(test_mma_w2a8)
ABQ_REF_STUB(test_mma_w3a3)
ABQ_REF_STUB(test_mma_w3a8)
ABQ_REF_STUB(test_mma_w4a4)
ABQ_REF_STUB(test_mma_w4a8)
ABQ_REF_STUB(test_mma_w5a5)
ABQ_REF_STUB(test_mma_w6a6)
ABQ_REF_STUB(test_mma_w7a7)
ABQ_REF_STUB(test_mma_w8a8)
