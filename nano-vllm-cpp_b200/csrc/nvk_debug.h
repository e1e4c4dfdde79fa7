/* Debug hooks of libnvk.so used by the tests; not part of the product ABI (include/nvk.h). */
#ifndef NVK_DEBUG_H
#define NVK_DEBUG_H
#ifdef __cplusplus
extern "C" {
#endif
/* When non-NULL, the next tcgen05 prefill launches copy the raw (unscaled) scores of the first
 * 128 x 128 tile of sequence 0, head 0 into this device buffer of 128 * 128 floats. */
void nvk_debug_set_prefill_dump(float* device_buffer);
/* When non-NULL, one block in the middle of the grid (head 0) stamps clock64() at seven points of each of
 * its first 64 key tiles into this device buffer of 64 * 8 int64 (phase timing of the prefill pipeline). */
void nvk_debug_set_prefill_clock(long long* device_buffer);
/* Returns and clears the error word a tcgen05 prefill block raises when a bounded wait times out
 * (0 = none; 1..6 = which wait).  Synchronises the device. */
int nvk_debug_take_device_error(void);
#ifdef __cplusplus
}
#endif
#endif
