"""Exception classes named after the TensorFlow status codes the reference op raises
(tf2/src/approx_nn_conv_ops.cpp:120-121,160-163,224-232,274-303; tf2/src/approx_ops_types.h:213)."""


class AxconvError(RuntimeError):
    code = -1


class InvalidArgumentError(AxconvError, ValueError):
    code = 3


class UnimplementedError(AxconvError, NotImplementedError):
    code = 12


class InternalError(AxconvError):
    code = 13


class CudaError(AxconvError):
    code = 100


_BY_CODE = {c.code: c for c in (InvalidArgumentError, UnimplementedError, InternalError, CudaError)}


def raise_for_status(status, what, detail=""):
    if status == 0:
        return
    cls = _BY_CODE.get(status, AxconvError)
    raise cls("%s: status %d%s" % (what, status, (" (" + detail + ")") if detail else ""))
