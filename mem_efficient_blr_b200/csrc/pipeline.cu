#include "pipeline.h"
#include "tmap.h"
namespace blr {
int pipeline_blast(const void*, int64_t, int64_t, int, const void*, int, const void*, int, const void*, int64_t, int64_t, int64_t, int, int, int, int, int, void*, int64_t, void*, void*, cudaStream_t) { set_last_error("pipeline not built"); return BLR_ERR_UNSUPPORTED; }
int pipeline_monarch(const void*, int64_t, int64_t, int, const void*, int, int, const void*, int, int, int, int, int, int, void*, int64_t, void*, cudaStream_t) { set_last_error("pipeline not built"); return BLR_ERR_UNSUPPORTED; }
int pipeline_low_rank(const void*, int64_t, int64_t, int, const void*, int, const void*, int, int, int, int, void*, int64_t, void*, cudaStream_t) { set_last_error("pipeline not built"); return BLR_ERR_UNSUPPORTED; }
int pipeline_dense(const void*, int64_t, int64_t, int, const void*, int, int, int, void*, int64_t, cudaStream_t) { set_last_error("pipeline not built"); return BLR_ERR_UNSUPPORTED; }
}
