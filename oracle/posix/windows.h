// POSIX stand-in for the few Win32 calls the reference engine's portable sources make (test infrastructure: used only to
// build the reference's own engine on Linux as the checker, never by the product).
// engine/src/engine.h:34,233,241,342 and engine/src/graph.cpp:37 probe for files with GetFileAttributesA;
// engine/src/graph.cpp:402 removes a hand-over file with DeleteFileA. The engine joins paths with '\\'
// (engine.h:231-236): both calls accept that separator and map it to '/'.
#pragma once
#include <strings.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>

typedef unsigned long DWORD;
#define INVALID_FILE_ATTRIBUTES ((DWORD)-1)
#define FILE_ATTRIBUTE_DIRECTORY 0x10
#define FILE_ATTRIBUTE_NORMAL 0x80

inline std::string kiln_posix_path(const char* p) {
    std::string s(p ? p : "");
    for (char& c : s)
        if (c == '\\') c = '/';
    return s;
}
inline DWORD GetFileAttributesA(const char* p) {
    struct stat st;
    if (stat(kiln_posix_path(p).c_str(), &st) != 0) return INVALID_FILE_ATTRIBUTES;
    return S_ISDIR(st.st_mode) ? FILE_ATTRIBUTE_DIRECTORY : FILE_ATTRIBUTE_NORMAL;
}
inline int DeleteFileA(const char* p) { return unlink(kiln_posix_path(p).c_str()) == 0; }
// engine.h:692, train_job.h:202, graph.cpp:143 compare checkpoint paths without case (an MSVC runtime name)
inline int _stricmp(const char* a, const char* b) { return strcasecmp(a, b); }
