/*
 * Developer entry points of libwm_b200.so.  Nothing here has a counterpart in the upstream project and no operator
 * of the package calls them; they exist for the tests and for looking into the pipelined kernels.
 */
#ifndef WM_B200_DEBUG_H
#define WM_B200_DEBUG_H

#include "wm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Pipeline event trace of the tcgen05 kernels.  Arms the trace for the launch after the next `arm_after` launches
 * (negative: disarm) and copies out the (tag, clock) pairs block (0,0,0) recorded so far; returns their count.
 * Always 0 unless the library was built with -DWM_B200_TRACE (python -m white_matter_b200.build --trace). */
WM_API int wm_debug_trace(long long* out, int capacity, int arm_after);

/* Makes a bounded wait of the pipelined kernels run out, the way it would if a hand-over between two roles were
 * ever lost: a one-block kernel waits on a barrier that nothing arrives on, with the wait's limit shortened to
 * `limit_ticks` clock ticks, gives up, records code 250 in the device status word (wm_device_status) and returns
 * normally -- no trap, no fault; the context stays usable.  Returns WM_OK when the launch was accepted. */
WM_API int wm_debug_expire_wait(long long limit_ticks, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WM_B200_DEBUG_H */
