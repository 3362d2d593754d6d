/*
 * openfish/openfish_error.h -- log-level control of the openfish C API.
 *
 * Drop-in for the reference header of the same name: the enumeration values and the two
 * functions below are what a caller of the reference links against
 * (reference include/openfish/openfish_error.h:45-55; the level lives in one process-wide
 * variable, default OPENFISH_LOG_VERB, reference src/error.c:33-41).
 * The reference header also carries printf-style logging macros for its own sources; they are
 * not part of the binary interface and are not reproduced here.
 */
#ifndef OPENFISH_ERROR_H
#define OPENFISH_ERROR_H

#ifdef __cplusplus
extern "C" {
#endif

/* How much the library writes to stderr.  Each level includes the ones above it. */
enum openfish_log_level_opt {
    OPENFISH_LOG_OFF,  /* nothing */
    OPENFISH_LOG_ERR,  /* errors */
    OPENFISH_LOG_WARN, /* + warnings */
    OPENFISH_LOG_INFO, /* + information */
    OPENFISH_LOG_VERB, /* + verbose (default) */
    OPENFISH_LOG_DBUG, /* + debugging */
    OPENFISH_LOG_TRAC  /* + tracing (one line per kernel launch) */
};

enum openfish_log_level_opt get_openfish_log_level(void);
void set_openfish_log_level(enum openfish_log_level_opt level);

#ifdef __cplusplus
}
#endif

#endif /* OPENFISH_ERROR_H */
