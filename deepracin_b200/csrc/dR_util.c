/*
 * Small host utilities: GLib stand-ins, the intrusive list of the graph core
 * (reference src/dR_core.c:504-665), string concatenation (:667-675) and the naive
 * matmuls used by host-side weight transforms (:677-723).
 */
#include <errno.h>
#include <stdarg.h>
#include <sys/stat.h>
#include <sys/types.h>
#include "dR_core.h"

gchar *dR_strdup_printf(const char *fmt, ...)
{
    va_list ap, ap2;
    va_start(ap, fmt);
    va_copy(ap2, ap);
    int n = vsnprintf(NULL, 0, fmt, ap);
    va_end(ap);
    gchar *s = (gchar *)malloc((size_t)n + 1);
    vsnprintf(s, (size_t)n + 1, fmt, ap2);
    va_end(ap2);
    return s;
}

gchar *dR_strdup(const char *s)
{
    if (!s) return NULL;
    size_t n = strlen(s) + 1;
    gchar *r = (gchar *)malloc(n);
    memcpy(r, s, n);
    return r;
}

gchar *dR_build_filename(const char *dir, const char *name)
{
    size_t n = strlen(dir);
    if (n > 0 && dir[n - 1] == '/') return dR_strdup_printf("%s%s", dir, name);
    return dR_strdup_printf("%s/%s", dir, name);
}

gchar *dR_file_get_contents(const char *path, size_t *length)
{
    FILE *fp = fopen(path, "rb");
    if (!fp) return NULL;
    fseek(fp, 0, SEEK_END);
    long n = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    gchar *buf = (gchar *)malloc((size_t)n + 1);
    if (fread(buf, 1, (size_t)n, fp) != (size_t)n) { fclose(fp); free(buf); return NULL; }
    fclose(fp);
    buf[n] = 0;
    if (length) *length = (size_t)n;
    return buf;
}

int dR_mkdir_with_parents(const char *path)
{
    gchar *tmp = dR_strdup(path);
    size_t n = strlen(tmp);
    for (size_t i = 1; i <= n; i++) {
        if (tmp[i] == '/' || tmp[i] == 0) {
            char keep = tmp[i];
            tmp[i] = 0;
            if (mkdir(tmp, 0777) != 0 && errno != EEXIST) { free(tmp); return -1; }
            tmp[i] = keep;
        }
    }
    free(tmp);
    return 0;
}

/* ------------------------------------------------------------------ list */
dR_List *dR_list_createEmptyList(void)
{
    dR_List *l = (dR_List *)calloc(1, sizeof(dR_List));
    return l;
}

void dR_list_append(dR_List *list, void *elem)
{
    dR_ListElement *e = (dR_ListElement *)calloc(1, sizeof(dR_ListElement));
    e->element = elem;
    e->previous = list->last;
    if (list->last) list->last->next = e; else list->first = e;
    list->last = e;
    list->length++;
}

gboolean dR_list_removeFirstOcc(dR_List *list, void *elem)
{
    for (dR_ListElement *e = list->first; e; e = e->next) {
        if (e->element != elem) continue;
        if (e->previous) e->previous->next = e->next; else list->first = e->next;
        if (e->next) e->next->previous = e->previous; else list->last = e->previous;
        if (list->iterator == e) list->iterator = e->next;
        free(e);
        list->length--;
        return TRUE;
    }
    return FALSE;
}

void *dR_list_pop(dR_List *list)
{
    dR_ListElement *e = list->first;
    if (!e) return NULL;
    void *r = e->element;
    list->first = e->next;
    if (e->next) e->next->previous = NULL; else list->last = NULL;
    if (list->iterator == e) list->iterator = e->next;
    free(e);
    list->length--;
    return r;
}

void *dR_list_next(dR_List *list)
{
    if (!list->iterator) return NULL;
    void *r = list->iterator->element;
    list->iterator = list->iterator->next;
    return r;
}

void dR_list_resetIt(dR_List *list) { list->iterator = list->first; }

void dR_list_cleanup(dR_List *list)
{
    if (!list) return;
    dR_ListElement *e = list->first;
    while (e) { dR_ListElement *n = e->next; free(e); e = n; }
    free(list);
}

gchar *concat_and_free_old(gchar *a, gchar *b)
{
    gchar *r = dR_strdup_printf("%s%s", a ? a : "", b ? b : "");
    free(a);
    free(b);
    return r;
}

gboolean dR_matmul(gfloat *m1, int r1, int c1, gfloat *m2, int r2, int c2, gfloat *res)
{
    if (c1 != r2) return FALSE;
    for (int i = 0; i < r1; i++)
        for (int j = 0; j < c2; j++) {
            gfloat s = 0.0f;
            for (int k = 0; k < c1; k++) s += m1[i * c1 + k] * m2[k * c2 + j];
            res[i * c2 + j] = s;
        }
    return TRUE;
}

gboolean dR_matmulT(gfloat *m1, int r1, int c1, gfloat *m2, int r2, int c2, gfloat *res)
{
    if (c1 != c2) return FALSE;
    for (int i = 0; i < r1; i++)
        for (int j = 0; j < r2; j++) {
            gfloat s = 0.0f;
            for (int k = 0; k < c1; k++) s += m1[i * c1 + k] * m2[j * c2 + k];
            res[i * r2 + j] = s;
        }
    return TRUE;
}
