/*
 * Minimal stand-ins for the GLib scalar types and helpers that deepRacin's public
 * headers use (the reference includes <glib.h>, include/dR_types.h:13).  Only the
 * names that appear in the public API and in this library's host code are provided.
 */
#ifndef DR_COMPAT_H
#define DR_COMPAT_H
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef int gint;
typedef int gboolean;
typedef float gfloat;
typedef double gdouble;
typedef char gchar;
typedef int32_t gint32;
typedef int64_t gint64;
typedef long glong;
typedef size_t gsize;
typedef unsigned int guint;
typedef void *gpointer;

#ifndef TRUE
#define TRUE 1
#endif
#ifndef FALSE
#define FALSE 0
#endif

#define g_malloc(n) malloc((size_t)(n))
#define g_malloc0(n) calloc(1, (size_t)(n))
#define g_free(p) free((void *)(p))
#define g_print(...) do { printf(__VA_ARGS__); fflush(stdout); } while (0)

#ifdef __cplusplus
extern "C" {
#endif
/* printf into a freshly malloc'ed string (g_strdup_printf). */
gchar *dR_strdup_printf(const char *fmt, ...);
gchar *dR_strdup(const char *s);
/* join directory and file name with exactly one '/' (g_build_filename for two parts). */
gchar *dR_build_filename(const char *dir, const char *name);
/* read a whole file; returns malloc'ed buffer (NUL terminated) or NULL (g_file_get_contents). */
gchar *dR_file_get_contents(const char *path, size_t *length);
/* mkdir -p; 0 on success (g_mkdir_with_parents). */
int dR_mkdir_with_parents(const char *path);
#ifdef __cplusplus
}
#endif
#define g_strdup_printf dR_strdup_printf
#define g_strdup dR_strdup
#endif
