"""The reference's own 19 tests (restated in tests/reference_suite.py) run
against the device host mirror: every value below is computed by the CUDA
kernels through the C ABI."""
import pytest

import reference_suite


@pytest.mark.gpu
@pytest.mark.parametrize("case", reference_suite.ALL, ids=lambda f: f.__name__)
def test_reference_case_on_device(case):
    import katsu_b200

    case(katsu_b200)


@pytest.mark.parametrize("case", reference_suite.NO_DEVICE, ids=lambda f: f.__name__)
def test_validation_needs_no_device(case):
    import katsu_b200

    case(katsu_b200)
