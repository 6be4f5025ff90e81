"""B200-native forward pass of TFApprox's `ApproxConv2DWithMinMaxVars` and a depthwise variant.

The compute lives in `libaxconv.so` (CUDA, sm_100a; C ABI in include/axconv.h).  This package is
the host-side mirror of the reference's Python-visible interface:

  approx_conv2d_with_min_max_vars(...)   same name and argument order as the op the reference
                                         registers (tf2/src/approx_nn_ops.cpp:38-54) and that its
                                         test calls (tf2/test/test_table_approx_conv_2d.py:46-49)
  FakeApproxConv2D                       the Keras layer of
                                         tf2/python/keras/layers/fake_approx_convolutional.py:176-261
"""
from .errors import InvalidArgumentError, UnimplementedError, InternalError, CudaError  # noqa: F401
from .tables import (exact_table, truncated_table, noisy_table, write_table, read_table,  # noqa: F401
                     table_from_function, table_from_c_source, table_report, tune_table, validate_table_file)
from .ops import (approx_conv2d_with_min_max_vars, approx_depthwise_conv2d_with_min_max_vars,  # noqa: F401
                  ax_conv2d, approx_conv2d,
                  conv2d_output_shape, launch_count, measure_lookup_peak, Table)
from .layers import FakeApproxConv2D, fake_quant_with_min_max_vars  # noqa: F401
