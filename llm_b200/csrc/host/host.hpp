// Shared by the files of the native host library (libllmb_host): error reporting across the
// C boundary. Functions are `extern "C"`, return LLMH_OK or a code below, and leave the text
// (and up to two numbers) of the calling thread's last failure to llmh_last_error(). The codes
// follow the engine error kinds of MythEclipse/llm (apps/engine/src/error.rs:9-17).
#pragma once

#include <cstdint>
#include <string>

#define LLMH_OK 0
#define LLMH_FORMAT 1         // a file or value that cannot be read as what it claims to be
#define LLMH_INVARIANT 2      // misuse or broken bookkeeping (a slot freed twice, ...)
#define LLMH_CACHE_FULL 3     // no free slot or page
#define LLMH_CONTEXT_FULL 4   // a sequence would outgrow its positions; numbers: used, capacity
#define LLMH_IO 5             // the operating system refused (open, map)

#define LLMH_EXPORT extern "C" __attribute__((visibility("default")))

namespace llmh {

struct Failure {
    int code;
    std::string text;
    long long first = 0, second = 0;
};

Failure& last_failure();                    // of the calling thread

// Runs `body`; a thrown Failure becomes the return code and the thread's last failure.
template <typename Body>
int guarded(Body body) {
    try {
        body();
        return LLMH_OK;
    } catch (const Failure& failure) {
        last_failure() = failure;
        return failure.code;
    } catch (const std::exception& error) {
        last_failure() = Failure{LLMH_INVARIANT, error.what()};
        return LLMH_INVARIANT;
    }
}

}  // namespace llmh
