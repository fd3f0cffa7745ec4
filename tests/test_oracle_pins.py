"""Pins the CPU oracle to the reference's own known answers: every #[test] of
crates/katsu-core/tests/{conv2d,autograd,tensor}.rs restated in
tests/reference_suite.py must pass on oracle/katsu_ref.py."""
import pytest

import reference_suite


@pytest.mark.parametrize("case", reference_suite.ALL, ids=lambda f: f.__name__)
def test_reference_case_on_oracle(oracle, case):
    case(oracle)
