// Replays the launches of one layer for the layers after it that are built alike.
//
// A step of a 36-layer model is about 290 launcher calls. Issued from Python one by one they cost
// more host time than the GPU needs for a step of a few hundred tokens. Layers that are built
// alike make the same calls with the same arguments, except for the addresses of their own
// tensors (weights, tables, cache planes). So the host records the calls of one layer, marks
// every argument that points into one of that layer's tensors as (slot, offset), and this file
// repeats the list for the following layers with the slots' addresses taken from a table:
// one call from Python for all of them. The launchers are the same functions with the same
// arguments; results are bit for bit those of the layer-by-layer path.
//
// Arguments travel as 64-bit words: integers and addresses as they are, floating-point
// arguments as the bits of a double.
#include <cstdint>
#include <cstring>
#include <type_traits>
#include <utility>

#include "launchers.h"

namespace {

template <class T>
inline T word_as(long long w) {
  if constexpr (std::is_pointer_v<T>) {
    return reinterpret_cast<T>(static_cast<uintptr_t>(w));
  } else if constexpr (std::is_floating_point_v<T>) {
    double d;
    memcpy(&d, &w, sizeof(d));
    return static_cast<T>(d);
  } else {
    return static_cast<T>(w);
  }
}

template <class... A, size_t... I>
inline int invoke(int (*fn)(A...), const long long* w, std::index_sequence<I...>) {
  return fn(word_as<A>(w[I])...);
}

template <class... A>
inline int call_with(int (*fn)(A...), const long long* w) {
  return invoke(fn, w, std::index_sequence_for<A...>{});
}

template <class... A>
constexpr int arity(int (*)(A...)) {
  return static_cast<int>(sizeof...(A));
}

struct Launcher {
  const char* name;
  int nargs;
  int (*call)(const long long*);
};

#define TIE_LAUNCHER(f) \
  { #f, arity(&f), [](const long long* w) -> int { return call_with(&f, w); } }

const Launcher kLaunchers[] = {
    TIE_LAUNCHER(tie_add_rmsnorm),          TIE_LAUNCHER(tie_rmsnorm_rows),         TIE_LAUNCHER(tie_silu_mul),
    TIE_LAUNCHER(tie_rope),                 TIE_LAUNCHER(tie_kv_append),            TIE_LAUNCHER(tie_qk_norm_rope_append),
    TIE_LAUNCHER(tie_gemm_simt),            TIE_LAUNCHER(tie_gemm_tc),              TIE_LAUNCHER(tie_gemm_tc2),
    TIE_LAUNCHER(tie_attention_rows),       TIE_LAUNCHER(tie_attention_split),      TIE_LAUNCHER(tie_attention_merge),
    TIE_LAUNCHER(tie_attention_prompt_tc),  TIE_LAUNCHER(tie_attention_decode_tc),  TIE_LAUNCHER(tie_attention_prompt_tma),
    TIE_LAUNCHER(tie_attention_decode_tma), TIE_LAUNCHER(tie_attention_prompt_umma), TIE_LAUNCHER(tie_attention_decode_prep),
};
constexpr int kNumLaunchers = static_cast<int>(sizeof(kLaunchers) / sizeof(kLaunchers[0]));
constexpr int kMaxArgs = 40;

}  // namespace

// The index of a launcher in the replay table, or -1 for a function that cannot be replayed.
TIE_API int tie_replay_launcher_id(const char* name) {
  for (int i = 0; i < kNumLaunchers; ++i)
    if (strcmp(kLaunchers[i].name, name) == 0) return i;
  return -1;
}

// How many arguments launcher `id` takes (-1 for a bad id).
TIE_API int tie_replay_launcher_args(int id) { return id >= 0 && id < kNumLaunchers ? kLaunchers[id].nargs : -1; }

// Repeats `n_calls` recorded calls for `n_layers` layers. Call c is launcher fn[c] with the words
// words[arg_begin[c] .. arg_begin[c + 1]); a word whose slot[] is s >= 0 is replaced, for layer l,
// by layer_ptrs[l * n_slots + s] + offset[]. Stops at the first call that fails and returns its
// status (its message is the launcher's); *failed_at receives layer * n_calls + call.
TIE_API int tie_replay_layers(const int* fn, const int* arg_begin, const long long* words, const int* slot,
                              const long long* offset, int n_calls, const long long* layer_ptrs, int n_slots,
                              int n_layers, int* failed_at) {
  TIE_REQUIRE(fn != nullptr && arg_begin != nullptr && words != nullptr && slot != nullptr && offset != nullptr &&
                  layer_ptrs != nullptr && n_calls >= 0 && n_slots >= 0 && n_layers >= 0,
              "layer replay: bad arguments (calls %d, slots %d, layers %d)", n_calls, n_slots, n_layers);
  for (int c = 0; c < n_calls; ++c) {
    const int id = fn[c], n = arg_begin[c + 1] - arg_begin[c];
    TIE_REQUIRE(id >= 0 && id < kNumLaunchers, "layer replay: call %d names launcher %d of %d", c, id, kNumLaunchers);
    TIE_REQUIRE(n == kLaunchers[id].nargs && n <= kMaxArgs, "layer replay: call %d gives %s %d arguments, it takes %d", c,
                kLaunchers[id].name, n, kLaunchers[id].nargs);
    for (int a = arg_begin[c]; a < arg_begin[c + 1]; ++a)
      TIE_REQUIRE(slot[a] < n_slots, "layer replay: argument %d of call %d names slot %d of %d", a - arg_begin[c], c,
                  slot[a], n_slots);
  }
  long long w[kMaxArgs];
  for (int l = 0; l < n_layers; ++l) {
    const long long* ptrs = layer_ptrs + static_cast<long long>(l) * n_slots;
    for (int c = 0; c < n_calls; ++c) {
      const int begin = arg_begin[c], n = arg_begin[c + 1] - begin;
      for (int a = 0; a < n; ++a) {
        const int s = slot[begin + a];
        w[a] = s >= 0 ? ptrs[s] + offset[begin + a] : words[begin + a];
      }
      const int status = kLaunchers[fn[c]].call(w);
      if (status != tie::kOk) {
        if (failed_at != nullptr) *failed_at = l * n_calls + c;
        return status;
      }
    }
  }
  return tie::kOk;
}
