#include <cstring>
#include "../../include/tile_sm100.h"
extern "C" {
const char* tsm100_target_name(void) { return "cuda_sm100"; }
const char* tsm100_target_ext(void) { return "cu"; }
int32_t tsm100_emit(const char*, size_t, char*, size_t, size_t*, char*, size_t, size_t*) { return TSM100_ERR_EMIT; }
}
