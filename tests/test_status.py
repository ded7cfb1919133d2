"""How a kernel's recorded failure reaches the caller (no GPU: the word's value is given).

Every wait inside the kernels is bounded; a wait that runs out writes a code into a status word on
the device and the kernel returns.  The host reads the word where it synchronises anyway (with the
sampled tokens, or in ``check_status``) and raises.  No test makes a kernel wait in vain: that would
occupy a GPU for seconds; what is tested here is the host's side of the path.
"""
import pytest

from rocml_b200 import kernels
from rocml_b200.errors import KernelError, RocmlError


def test_zero_is_no_failure():
    kernels.raise_for_status(0)


@pytest.mark.parametrize("code,word", [(10004, "wait"), (10001, "size")])
def test_a_recorded_code_raises_with_its_meaning(code, word):
    with pytest.raises(KernelError) as e:
        kernels.raise_for_status(code)
    assert str(code) in str(e.value) and word in str(e.value).lower()
    assert isinstance(e.value, RocmlError)


def test_an_unknown_code_still_raises():
    with pytest.raises(KernelError, match="code 77"):
        kernels.raise_for_status(77)
