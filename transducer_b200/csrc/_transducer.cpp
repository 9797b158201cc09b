// pybind11 module `_transducer`: the Python <-> C++ boundary.
//
// Exposes the three functions of the reference's shim under the same names and
// keyword arguments (transducer/_transducer.cpp:9-148 -- pointers travel as integers
// obtained from tensor.data_ptr()), plus the entry points of transducer_b200.h that
// replace the torch-op arithmetic of transducer/torch_binding.py.  Failures surface as
// ValueError (invalid argument) or RuntimeError (CUDA), as pybind11 maps the
// reference's std::invalid_argument / std::runtime_error.
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/transducer.h"
#include "../../include/transducer_b200.h"

namespace py = pybind11;
using namespace py::literals;
using addr = std::uintptr_t;

namespace {

template <typename T>
T* at(addr a) { return reinterpret_cast<T*>(a); }

void check(int rc) {
  if (rc == TB200_OK) return;
  if (rc == TB200_ERR_INVALID_ARGUMENT || rc == TB200_ERR_WORKSPACE)
    throw std::invalid_argument(tb200_last_error());
  throw std::runtime_error(tb200_last_error());
}

}  // namespace

PYBIND11_MODULE(_transducer, m) {
  m.doc() = "sm_100a RNN-T loss / Viterbi kernels (drop-in for awni/transducer's _transducer)";

  // ---- reference-compatible trio -------------------------------------------------
  m.def("forward",
        [](addr e, addr p, addr costs, addr alphas, addr ln, addr labels, addr ilen, addr llen,
           int B, int T, int U, int V, int blank, bool use_cuda) {
          forward(at<const float>(e), at<const float>(p), at<float>(costs), at<float>(alphas),
                  at<const float>(ln), at<const int>(labels), at<const int>(ilen),
                  at<const int>(llen), B, T, U, V, blank, use_cuda);
        },
        "emissions"_a, "predictions"_a, "costs"_a, "alphas"_a, "logNorms"_a, "labels"_a,
        "input_lengths"_a, "label_lengths"_a, "batch_size"_a, "max_input_length"_a,
        "max_label_length"_a, "alphabet_size"_a, "blank"_a, "use_cuda"_a);

  m.def("backward",
        [](addr e, addr p, addr eg, addr pg, addr lg, addr alphas, addr ln, addr labels,
           addr ilen, addr llen, int B, int T, int U, int V, int blank, bool use_cuda) {
          backward(at<const float>(e), at<const float>(p), at<float>(eg), at<float>(pg),
                   at<float>(lg), at<const float>(alphas), at<const float>(ln),
                   at<const int>(labels), at<const int>(ilen), at<const int>(llen), B, T, U, V,
                   blank, use_cuda);
        },
        "emissions"_a, "predictions"_a, "egrads"_a, "pgrads"_a, "lngrads"_a, "alphas"_a,
        "logNorms"_a, "labels"_a, "input_lengths"_a, "label_lengths"_a, "batch_size"_a,
        "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a, "blank"_a,
        "use_cuda"_a);

  m.def("viterbi",
        [](addr e, addr p, addr ln, addr labels, addr ilen, addr llen, int B, int T, int U,
           int V, int blank, bool use_cuda) {
          viterbi(at<const float>(e), at<const float>(p), at<const float>(ln), at<int>(labels),
                  at<const int>(ilen), at<const int>(llen), B, T, U, V, blank, use_cuda);
        },
        "emissions"_a, "predictions"_a, "log_norms"_a, "labels"_a, "input_lengths"_a,
        "label_lengths"_a, "batch_size"_a, "max_input_length"_a, "max_label_length"_a,
        "alphabet_size"_a, "blank"_a, "use_cuda"_a);

  // ---- fused path ------------------------------------------------------------------
  m.def("set_stream", [](addr s) { check(tb200_set_stream(at<void>(s))); }, "stream"_a);
  m.def("set_option", [](const char* k, int v) { check(tb200_set_option(k, v)); }, "key"_a,
        "value"_a);
  m.def("get_option", [](const char* k) { int v = 0; check(tb200_get_option(k, &v)); return v; },
        "key"_a);

  m.def("log_norms_workspace_bytes", &tb200_log_norms_workspace_bytes);
  m.def("loss_forward_workspace_bytes", &tb200_loss_forward_workspace_bytes);
  m.def("loss_backward_workspace_bytes", &tb200_loss_backward_workspace_bytes);
  m.def("viterbi_decode_workspace_bytes", &tb200_viterbi_decode_workspace_bytes);

  m.def("log_norms",
        [](addr e, addr p, addr ln, addr rowref, addr maxp, addr ilen, addr llen, int B, int T,
           int U, int V, addr ws, size_t wsBytes) {
          check(tb200_log_norms(at<const float>(e), at<const float>(p), at<float>(ln),
                                at<float>(rowref), at<float>(maxp), at<const int>(ilen),
                                at<const int>(llen), B, T, U, V, at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "log_norms"_a, "row_ref"_a, "max_p"_a,
        "input_lengths"_a, "label_lengths"_a, "batch_size"_a, "max_input_length"_a,
        "max_label_length"_a, "alphabet_size"_a, "workspace"_a, "workspace_bytes"_a);

  m.def("loss_saved_bytes", &tb200_loss_saved_bytes);

  m.def("loss_forward",
        [](addr e, addr p, addr labels, addr ilen, addr llen, addr costs, addr loss_sum,
           addr saved, size_t savedBytes, int B, int T, int U, int V, int blank, addr ws,
           size_t wsBytes) {
          check(tb200_loss_forward(at<const float>(e), at<const float>(p), at<const int>(labels),
                                   at<const int>(ilen), at<const int>(llen), at<float>(costs),
                                   at<float>(loss_sum), at<void>(saved), savedBytes, B, T, U, V,
                                   blank, at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "labels"_a, "input_lengths"_a, "label_lengths"_a,
        "costs"_a, "loss_sum"_a, "saved"_a, "saved_bytes"_a, "batch_size"_a,
        "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a, "blank"_a, "workspace"_a,
        "workspace_bytes"_a);

  m.def("loss_forward_bf16",
        [](addr e, addr p, addr labels, addr ilen, addr llen, addr costs, addr loss_sum,
           addr saved, size_t savedBytes, int B, int T, int U, int V, int blank, addr ws,
           size_t wsBytes) {
          check(tb200_loss_forward_bf16(at<const void>(e), at<const void>(p),
                                        at<const int>(labels), at<const int>(ilen),
                                        at<const int>(llen), at<float>(costs), at<float>(loss_sum),
                                        at<void>(saved), savedBytes, B, T, U, V, blank,
                                        at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "labels"_a, "input_lengths"_a, "label_lengths"_a,
        "costs"_a, "loss_sum"_a, "saved"_a, "saved_bytes"_a, "batch_size"_a,
        "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a, "blank"_a, "workspace"_a,
        "workspace_bytes"_a);

  m.def("loss_backward_bf16",
        [](addr e, addr p, addr labels, addr ilen, addr llen, addr saved, size_t savedBytes,
           addr deltas, addr eg, addr pg, int B, int T, int U, int V, int blank, addr ws,
           size_t wsBytes) {
          check(tb200_loss_backward_bf16(at<const void>(e), at<const void>(p),
                                         at<const int>(labels), at<const int>(ilen),
                                         at<const int>(llen), at<const void>(saved), savedBytes,
                                         at<const float>(deltas), at<void>(eg), at<void>(pg), B,
                                         T, U, V, blank, at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "labels"_a, "input_lengths"_a, "label_lengths"_a,
        "saved"_a, "saved_bytes"_a, "deltas"_a, "egrads"_a, "pgrads"_a, "batch_size"_a,
        "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a, "blank"_a, "workspace"_a,
        "workspace_bytes"_a);

  m.def("loss_backward",
        [](addr e, addr p, addr labels, addr ilen, addr llen, addr saved, size_t savedBytes,
           addr deltas, addr eg, addr pg, int B, int T, int U, int V, int blank, addr ws,
           size_t wsBytes) {
          check(tb200_loss_backward(at<const float>(e), at<const float>(p),
                                    at<const int>(labels), at<const int>(ilen),
                                    at<const int>(llen), at<const void>(saved), savedBytes,
                                    at<const float>(deltas), at<float>(eg), at<float>(pg), B, T,
                                    U, V, blank, at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "labels"_a, "input_lengths"_a, "label_lengths"_a,
        "saved"_a, "saved_bytes"_a, "deltas"_a, "egrads"_a, "pgrads"_a, "batch_size"_a,
        "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a, "blank"_a, "workspace"_a,
        "workspace_bytes"_a);

  m.def("viterbi_decode",
        [](addr e, addr p, addr ilen, addr llen, addr labels, int B, int T, int U, int V,
           int blank, addr ws, size_t wsBytes) {
          check(tb200_viterbi_decode(at<const float>(e), at<const float>(p), at<const int>(ilen),
                                     at<const int>(llen), at<int>(labels), B, T, U, V, blank,
                                     at<void>(ws), wsBytes));
        },
        "emissions"_a, "predictions"_a, "input_lengths"_a, "label_lengths"_a, "labels"_a,
        "batch_size"_a, "max_input_length"_a, "max_label_length"_a, "alphabet_size"_a,
        "blank"_a, "workspace"_a, "workspace_bytes"_a);

  // ---- device status (bounded waits that ran out) -----------------------------------
  // Returns the code of tb200_check_status (0, or 5 = a kernel gave up) without throwing, so the
  // Python layer can raise its own exception type; the text is in last_error().
  m.def("check_status", []() { return tb200_check_status(); });
  m.def("last_error", []() { return std::string(tb200_last_error()); });
  m.def("status_name", [](int code) { return std::string(tb200_status_name(code)); }, "code"_a);
  m.def("selftest_wait_timeout",
        [](unsigned us) { check(tb200_selftest_wait_timeout(us)); }, "limit_microseconds"_a);

  m.attr("__version__") = "b200-" + std::to_string(tb200_version());
}
