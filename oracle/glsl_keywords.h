// Test infrastructure only. Include AFTER every other header and immediately
// before the reference shaders: these macros turn GLSL storage qualifiers into
// C++ ones and restate what Program::GetHead prepends to every shader
// (ogl_runtime/opengl/core/program.cc:92-102).
#ifndef ORACLE_GLSL_KEYWORDS_H_
#define ORACLE_GLSL_KEYWORDS_H_
#define PRECISION
#define highp
// 1-D ("ANY4") tensors wrap at this many texels per row. It is chosen larger
// than any tensor used here so that every 1-D tensor is a single row and
// pos.y stays 0.
#define MAX_TEXTURE_SIZE 268435456
#define uniform static
#define out static thread_local
#endif  // ORACLE_GLSL_KEYWORDS_H_
