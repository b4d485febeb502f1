/* The reference tokenizer includes <pcre2posix.h> but uses nothing from it; an empty header is enough. */
#ifndef CVERL_B200_BASELINE_PCRE2POSIX_SHIM_H_
#define CVERL_B200_BASELINE_PCRE2POSIX_SHIM_H_
#endif
