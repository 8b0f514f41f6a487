// POSIX stand-in for <io.h>: engine/src/main.cpp:621 switches stdout to binary mode, which is what a POSIX stream already is.
#pragma once
#include <cstdio>
#ifndef _O_BINARY
#define _O_BINARY 0
#endif
inline int _fileno(FILE* f) { return fileno(f); }
inline int _setmode(int, int) { return 0; }
