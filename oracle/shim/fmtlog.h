// Build shim for the reference oracle: logging macros become no-ops (fmtlog is not vendored).
#pragma once
#include <fmt/format.h>
#define logd(...) ((void) 0)
#define logi(...) ((void) 0)
#define logw(...) ((void) 0)
#define loge(...) ((void) 0)
namespace fmtlog {
    enum LogLevel { DBG, INF, WRN, ERR, OFF };
    inline void setLogLevel(LogLevel) {}
    inline void setLogFile(const char *, bool = false) {}
    inline void startPollingThread(long = 0) {}
    inline void poll(bool = false) {}
}// namespace fmtlog
