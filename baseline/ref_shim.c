/* The reference's CUDA translation units report errors through one host function that lives in its main host source.
 * That source does not compile against CUDA 12.9 (it passes const arrays to a copy routine whose parameters lost their
 * const qualifiers, and appends a stream argument the routine no longer takes), so the kernel objects are linked with
 * this sink instead: the last message is kept and can be read back. */
#include <string.h>

static char last_message[512];

void ds41rt_set_last_error_message(const char* message) {
  if (!message) { last_message[0] = 0; return; }
  strncpy(last_message, message, sizeof(last_message) - 1);
  last_message[sizeof(last_message) - 1] = 0;
}

const char* ds41rt_ref_shim_last_message(void) { return last_message; }
