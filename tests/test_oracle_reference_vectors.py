"""The CPU oracle against the reference's own known-answer vectors (no GPU)."""
import pytest

import reference_cases as rc


@pytest.mark.parametrize("case", rc.FOLD_CASES + rc.TABLE_CASES, ids=lambda c: c.__name__)
def test_oracle_matches_reference_vector(case, oracle):
    case(oracle)


@pytest.mark.parametrize("case", rc.FOLD_CASES + rc.TABLE_CASES, ids=lambda c: c.__name__)
def test_oracle_threaded_matches_reference_vector(case, oracle_mt):
    case(oracle_mt)
