"""Builds the reference's own pybind module on top of libcs2d.so.

The reference's host file ``kernels/selective_nd_scan/src/cusoflex/selective_scan_oflex.cpp``
validates the tensors, allocates the outputs and dispatches to its CUDA kernels.  This script
shows - and tests - the edit a maintainer of the reference makes to keep that file (its checks,
its pybind module ``selective_nd_scan_cuda_oflex`` with ``fwd`` / ``bwd``, unchanged signatures)
and run this library's kernels underneath:

* the side-buffer allocations (``x``, ``x_v``, ``x_sd``, lines 251-258) and ``set_ssm_params_fwd``
  become one ``x_v`` of ``cs2d_saved_bytes`` and two empty tensors;
* the forward dispatch block (lines 275-281) becomes ``cs2d_fwd``;
* the shape checks of the three saved tensors in ``selective_scan_bwd`` (lines 367-391: they
  describe the reference kernels' private layouts) become a size check of ``x_v``;
* ``set_ssm_params_bwd`` and the backward dispatch block (lines 424-430) become ``cs2d_bwd``.

Nothing of the reference is stored in this repository: the script reads the host file from a
checkout of the reference, writes the edited copy into ``tests/integration/_build/`` (not under
version control), compiles it with g++ against torch and ``libcs2d.so`` into the module
``tests/integration/_build/selective_nd_scan_cuda_oflex.so`` and deletes the copy again.

    python tests/integration/make_binding.py /path/to/official-cross-scan
"""
import os
import re
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build")
LIBDIR = os.path.join(ROOT, "official-cross-scan_b200", "cs2d")

HELPER = r'''
#include "cs2d.h"   // this library's C ABI; link with libcs2d.so

static cs2d_problem cs2d_make_problem(const at::Tensor &u, const at::Tensor &delta, const at::Tensor &A,
                                      const at::Tensor &B, const at::Tensor &C, const void *D, const void *bias,
                                      const void *decay, bool softplus, at::ScalarType out_type) {
    auto dt = [](at::ScalarType t) { return t == at::kFloat ? CS2D_F32 : t == at::kHalf ? CS2D_F16 : CS2D_BF16; };
    cs2d_problem p{};
    p.batch = u.size(0); p.dim = u.size(1); p.nrows = u.size(2); p.ncols = u.size(3);
    p.dstate = A.size(1); p.n_groups = B.size(1); p.delta_dim = delta.size(1);
    p.io_dtype = dt(u.scalar_type()); p.out_dtype = dt(out_type); p.delta_softplus = softplus;
    p.u = u.data_ptr();         p.u_bs = u.stride(0);         p.u_ds = u.stride(1);         p.u_hs = u.stride(2);
    p.delta = delta.data_ptr(); p.delta_bs = delta.stride(0); p.delta_ds = delta.stride(1); p.delta_hs = delta.stride(2);
    p.A = A.data_ptr<float>();  p.A_ds = A.stride(0);         p.A_ns = A.stride(1);
    p.B = B.data_ptr(); p.B_bs = B.stride(0); p.B_gs = B.stride(1); p.B_ns = B.stride(2); p.B_hs = B.stride(3);
    p.C = C.data_ptr(); p.C_bs = C.stride(0); p.C_gs = C.stride(1); p.C_ns = C.stride(2); p.C_hs = C.stride(3);
    p.D = (const float *)D; p.delta_bias = (const float *)bias; p.A_decay = (const float *)decay;
    return p;
}
'''

FWD_ALLOC = r'''
    at::cuda::CUDAGuard cs2d_guard{(char)u.get_device()};
    cs2d_problem cs2d_p = cs2d_make_problem(u, delta, A, B, C,
        D_.has_value() ? D_.value().data_ptr() : nullptr,
        delta_bias_.has_value() ? delta_bias_.value().data_ptr() : nullptr,
        A_decay_.has_value() ? A_decay_.value().data_ptr() : nullptr, delta_softplus, out.scalar_type());
    const size_t cs2d_nsaved = cs2d_saved_bytes(&cs2d_p);
    TORCH_CHECK(cs2d_nsaved > 0, cs2d_last_error());
    at::Tensor x_v = torch::empty({(int64_t)(cs2d_nsaved / 4)}, u.options().dtype(weight_type));
    at::Tensor x = torch::empty({0}, x_v.options()), x_sd = torch::empty({0}, x_v.options());
'''

FWD_CALL = r'''
    TORCH_CHECK(cs2d_fwd(&cs2d_p, out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), x_v.data_ptr(),
                         stream) == 0, cs2d_last_error());
'''

BWD_CHECK = r'''
    TORCH_CHECK(x_v_.has_value(), "the saved state x_v returned by fwd is required");
    {
        auto x_v = x_v_.value();
        TORCH_CHECK(x_v.scalar_type() == weight_type);
        TORCH_CHECK(x_v.is_cuda());
        TORCH_CHECK(x_v.is_contiguous());
    }
'''

BWD_CALL = r'''
    at::cuda::CUDAGuard device_guard{(char)u.get_device()};
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    cs2d_problem cs2d_p = cs2d_make_problem(u, delta, A, B, C,
        D_.has_value() ? D_.value().data_ptr() : nullptr,
        delta_bias_.has_value() ? delta_bias_.value().data_ptr() : nullptr,
        A_decay_.has_value() ? A_decay_.value().data_ptr() : nullptr, delta_softplus, dout.scalar_type());
    TORCH_CHECK((size_t)x_v_.value().numel() * 4 == cs2d_saved_bytes(&cs2d_p), "x_v is not the saved state fwd returned for these inputs");
    at::Tensor cs2d_scratch = torch::empty({(int64_t)(cs2d_bwd_scratch_bytes(&cs2d_p) / 4)}, u.options().dtype(at::kFloat));
    TORCH_CHECK(cs2d_bwd(&cs2d_p, dout.data_ptr(), dout.stride(0), dout.stride(1), dout.stride(2),
                         x_v_.value().data_ptr(), cs2d_scratch.data_ptr(), du.data_ptr(), ddelta.data_ptr(),
                         dA.data_ptr<float>(), dB.data_ptr<float>(), dC.data_ptr<float>(),
                         D_.has_value() ? dD.data_ptr<float>() : nullptr,
                         delta_bias_.has_value() ? ddelta_bias.data_ptr<float>() : nullptr,
                         A_decay_.has_value() ? dA_decay.data_ptr<float>() : nullptr, stream) == 0, cs2d_last_error());
'''


def sub_once(pattern, repl, text, what):
    new, n = re.subn(pattern, lambda m: repl, text, count=0, flags=re.S)
    if n != 1:
        raise SystemExit(f"make_binding: expected exactly one place for the {what}, found {n} - has the reference changed?")
    return new


def edit(src):
    """The five edits described in the module docstring, each anchored on the reference's own text."""
    src = sub_once(r'(#include "selective_scan_common\.h"\n)', '#include "selective_scan_common.h"\n' + HELPER, src,
                   "include block")
    # forward: side buffers + parameter struct  ->  one saved-state tensor
    src = sub_once(r'    at::Tensor x = torch::empty\(\{batch_size, dim, dstate, nChunksX, nrows \* 2\}.*?'
                   r'    SSMParamsBase params;\n    set_ssm_params_fwd\(.*?\n    \);\n', FWD_ALLOC, src,
                   "forward side-buffer allocation")
    src = sub_once(r'    DISPATCH_ITYPE_FLOAT_AND_HALF_AND_BF16\(u\.scalar_type\(\), "selective_scan_fwd", \[&\] \{.*?\n    \}\);\n',
                   FWD_CALL, src, "forward dispatch block")
    # backward: layout checks of the saved tensors  ->  a size check; parameter struct + dispatch  ->  cs2d_bwd
    src = sub_once(r'    if \(nChunksX > 1 \|\| nChunksY > 1\) \{ TORCH_CHECK\(x_\.has_value\(\)\); \}.*?'
                   r'CHECK_SHAPE\(x_v, batch_size, dim, dstate, nChunksY, ncols\);\s*\n    \}\n', BWD_CHECK, src,
                   "backward saved-tensor checks")
    src = sub_once(r'    SSMParamsBwd params;\n    set_ssm_params_bwd\(.*?'
                   r'    DISPATCH_ITYPE_FLOAT_AND_HALF_AND_BF16\(u\.scalar_type\(\), "selective_scan_bwd", \[&\] \{.*?\n    \}\);\n',
                   BWD_CALL, src, "backward dispatch block")
    return src


def build(ref):
    import torch
    r = os.path.join(ref, "kernels", "selective_nd_scan")
    host = os.path.join(r, "src", "cusoflex", "selective_scan_oflex.cpp")
    with open(host) as f:
        src = edit(f.read())
    os.makedirs(OUT, exist_ok=True)
    cpp = os.path.join(OUT, "selective_scan_oflex_on_cs2d.cpp")
    with open(cpp, "w") as f:
        f.write(src)
    tdir = os.path.dirname(torch.__file__)
    so = os.path.join(OUT, "selective_nd_scan_cuda_oflex.so")
    cmd = ["g++", "-shared", "-o", so, cpp, "-O2", "-std=c++17", "-fPIC", "-w",
           f"-I{r}/include", f"-I{r}/include/cusoflex", f"-I{ROOT}/include",
           f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include", f"-I{sysconfig.get_paths()['include']}",
           "-I/usr/local/cuda/include", "-DTORCH_EXTENSION_NAME=selective_nd_scan_cuda_oflex",
           "-D_GLIBCXX_USE_CXX11_ABI=1", f"-L{tdir}/lib", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           "-ltorch_python", f"-L{LIBDIR}", "-l:libcs2d.so", f"-Wl,-rpath,{tdir}/lib", "-Wl,-rpath,$ORIGIN/../../../official-cross-scan_b200/cs2d"]
    try:
        subprocess.run(cmd, check=True)
    finally:
        os.remove(cpp)   # the edited copy of the reference's file is a build intermediate only
    return so


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1]))
