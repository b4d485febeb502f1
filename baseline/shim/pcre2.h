/* Prototype-only stand-in for <pcre2.h>, 8-bit code units.
 *
 * The image ships the PCRE2 runtime (libpcre2-8.so.0) without its development header.
 * The unmodified reference tokenizer (src/text/hf_bpe_tokenizer.cc:3-7,138-196) uses seven
 * functions and two option bits of the documented public API; they are declared here with the
 * `_8` suffixed symbol names the 8-bit library exports, so that translation unit compiles
 * without any change and links against the runtime library.
 */
#ifndef CVERL_B200_BASELINE_PCRE2_SHIM_H_
#define CVERL_B200_BASELINE_PCRE2_SHIM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint8_t PCRE2_UCHAR8;
typedef const PCRE2_UCHAR8* PCRE2_SPTR8;
typedef size_t PCRE2_SIZE;
#define PCRE2_UCHAR PCRE2_UCHAR8
#define PCRE2_SPTR PCRE2_SPTR8

#define PCRE2_UCP 0x00020000u
#define PCRE2_UTF 0x00080000u

struct pcre2_real_code_8;
struct pcre2_real_match_data_8;
struct pcre2_real_compile_context_8;
struct pcre2_real_general_context_8;
struct pcre2_real_match_context_8;
typedef struct pcre2_real_code_8 pcre2_code_8;
typedef struct pcre2_real_match_data_8 pcre2_match_data_8;
typedef struct pcre2_real_compile_context_8 pcre2_compile_context_8;
typedef struct pcre2_real_general_context_8 pcre2_general_context_8;
typedef struct pcre2_real_match_context_8 pcre2_match_context_8;
#define pcre2_code pcre2_code_8
#define pcre2_match_data pcre2_match_data_8

pcre2_code_8* pcre2_compile_8(PCRE2_SPTR8, PCRE2_SIZE, uint32_t, int*, PCRE2_SIZE*, pcre2_compile_context_8*);
void pcre2_code_free_8(pcre2_code_8*);
int pcre2_get_error_message_8(int, PCRE2_UCHAR8*, PCRE2_SIZE);
pcre2_match_data_8* pcre2_match_data_create_from_pattern_8(const pcre2_code_8*, pcre2_general_context_8*);
void pcre2_match_data_free_8(pcre2_match_data_8*);
int pcre2_match_8(const pcre2_code_8*, PCRE2_SPTR8, PCRE2_SIZE, PCRE2_SIZE, uint32_t, pcre2_match_data_8*,
                  pcre2_match_context_8*);
PCRE2_SIZE* pcre2_get_ovector_pointer_8(pcre2_match_data_8*);

#define pcre2_compile pcre2_compile_8
#define pcre2_code_free pcre2_code_free_8
#define pcre2_get_error_message pcre2_get_error_message_8
#define pcre2_match_data_create_from_pattern pcre2_match_data_create_from_pattern_8
#define pcre2_match_data_free pcre2_match_data_free_8
#define pcre2_match pcre2_match_8
#define pcre2_get_ovector_pointer pcre2_get_ovector_pointer_8

#ifdef __cplusplus
}
#endif
#endif
