// One thread-local error text for the whole library.  Every extern "C" entry point that returns a
// non-zero tdc_status first records why through tdc::fail, and tdc_last_error_string() (and its older
// alias tdc_tc_last_error_string()) hands that text to the caller.  The reference drivers print and
// exit(-1) instead (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:31-47).
#pragma once

namespace tdc {

// Records the formatted message for the calling thread and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
const char* last_error();

}  // namespace tdc
