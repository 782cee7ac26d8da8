// Bindings of the peer-to-peer kernels.
#include <torch/extension.h>

void bind_p2p(pybind11::module& m) { (void)m; }
