// Levelled logger.  MINI_NCCL_DEBUG = NONE | WARN (default) | INFO | TRACE.
// The reference prints unconditionally with bracketed tags (reference:
// src/api.cpp:39,48,63; include/Config.h:56); the same tags are kept, the
// level gate is new.
#pragma once
#include <cstdarg>
#include <cstdio>

namespace mnccl {

enum class LogLevel : int { None = 0, Warn = 1, Info = 2, Trace = 3 };

LogLevel log_level();
void set_log_level(LogLevel lvl);
// Always printed (banner-type lines the reference prints unconditionally),
// unless the level is None.
void log_always(const char* tag, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void log_at(LogLevel lvl, const char* tag, const char* fmt, ...)
    __attribute__((format(printf, 3, 4)));

#define MNCCL_WARN(tag, ...) ::mnccl::log_at(::mnccl::LogLevel::Warn, tag, __VA_ARGS__)
#define MNCCL_INFO(tag, ...) ::mnccl::log_at(::mnccl::LogLevel::Info, tag, __VA_ARGS__)
#define MNCCL_TRACE(tag, ...) ::mnccl::log_at(::mnccl::LogLevel::Trace, tag, __VA_ARGS__)

}  // namespace mnccl
