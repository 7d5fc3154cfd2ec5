"""The host half of the kernels' status word, which needs no GPU: which code means what, and that a code is an error."""

import pytest


def test_kernel_status_codes_are_told_apart():
    from stride_b200.csrc import ops
    ops.raise_on_kernel_status(0)
    for code, text in ((1, "producer"), (2, "tensor-core issuer"), (3, "epilogue"), (15, "prefill attention"),
                       (31, "decode attention"), (32, "context bound"), (41, "weight-streaming"), (77, "unknown place")):
        with pytest.raises(ops.KernelError, match=text):
            ops.raise_on_kernel_status(code)


def test_the_status_word_of_a_device_that_was_never_used_reads_zero():
    from stride_b200.csrc import ops
    assert ops.tc_status("cuda:7") == 0
    ops.reset_kernel_status("cuda:7")       # nothing to clear, no error
