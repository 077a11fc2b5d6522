// Library-wide entry points: version, error text, table validation.
#include <string.h>

#include "jqk_common.cuh"

namespace jqk {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int32_t check_tables(const jqk_head_tables* t) {
  if (!t) return fail(JQK_E_ARG, "null head tables");
  if (t->n_heads <= 0 || t->n_heads > 1024) return fail(JQK_E_ARG, "n_heads %d out of range", t->n_heads);
  if (t->d <= 0 || t->d > JQK_MAX_DIM || t->d % 16) return fail(JQK_E_UNSUPPORTED, "head_dim %d must be a multiple of 16 and at most %d", t->d, JQK_MAX_DIM);
  if (t->words_per_record <= 0 || t->words_per_record > JQK_MAX_WORDS) return fail(JQK_E_LAYOUT, "words_per_record %d outside 1..%d", t->words_per_record, JQK_MAX_WORDS);
  if (!t->desc || !t->col_meta || !t->table_fields || !t->fwd_cols || !t->thresholds || !t->cb_cols ||
      !t->qproj_cols || !t->inv_rows)
    return fail(JQK_E_ARG, "head tables hold a null pointer");
  if (t->n_wide < 0 || t->n_wide > JQK_MAX_WIDE) return fail(JQK_E_LAYOUT, "n_wide %d outside 0..%d", t->n_wide, JQK_MAX_WIDE);
  if (t->n_wide > 0 && (!t->wide_thr || !t->wide_cb)) return fail(JQK_E_ARG, "tables with wide columns need wide_thr and wide_cb");
  return 0;
}

// The score and decode kernels keep all lookup tables of a head in shared memory.
int32_t check_decodable(const jqk_head_tables* t, const char* what) {
  if (t && t->n_wide > 0 && !t->decodable)
    return fail(JQK_E_UNSUPPORTED, "%s: the lookup tables of a head do not fit (%d columns above 4 bits take 2..16 table slots each)", what, t->n_wide);
  return 0;
}

}  // namespace jqk

extern "C" int32_t jqk_version(void) { return JQK_VERSION; }

extern "C" size_t jqk_head_tables_bytes(void) { return sizeof(jqk_head_tables); }

extern "C" const char* jqk_last_error(void) { return jqk::error_buffer(); }
