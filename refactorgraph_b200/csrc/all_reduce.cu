// placeholder until the peer-memory all-reduce lands
#include "gemm_dispatch.cuh"
namespace rg {
int all_reduce_error_word() { return 0; }
}// namespace rg
extern "C" {
int rg_b200_comm_create(int, int, size_t, rg_comm **, void *) { return RG_ERR_UNSUPPORTED; }
int rg_b200_comm_connect(rg_comm *, const void *) { return RG_ERR_UNSUPPORTED; }
int rg_b200_comm_status(rg_comm *) { return RG_ERR_UNSUPPORTED; }
int rg_b200_comm_destroy(rg_comm *) { return RG_ERR_UNSUPPORTED; }
int rg_b200_all_reduce(rg_comm *, const rg_all_reduce_params *, const void *const *, void *const *, void *) { return RG_ERR_UNSUPPORTED; }
}
