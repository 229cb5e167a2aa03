"""The greedy pick for callers that cannot allocate (`btb_b200_argmax_bf16_static`): a host that was granted its device
memory once at start-up, or code inside a stream capture, cannot create the scratch buffer the ordinary pick wants, so
this variant keeps its scratch inside the library. It must pick exactly what the ordinary entry point picks - token ids
are integers, so the comparison is equality - twice in a row (the shared scratch has to come back clean), whether this
file runs alone in a fresh process or after every other test."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402


def test_static_scratch_pick_equals_the_ordinary_pick_twice():
    rng = np.random.default_rng(12)
    for T, V in ((1, 151936), (7, 4099), (32, 2048)):
        lg = torch.from_numpy(rng.standard_normal((T, V)).astype(np.float32)).to(torch.bfloat16).cuda()
        lg[:, V // 3] = lg.max() + 1  # a planted tie at the top: the lowest index must win in both
        lg[:, V // 2] = lg[:, V // 3]
        scratch = torch.zeros(int(capi.lib().btb_b200_argmax_scratch_bytes(T)) // 8 + 1, dtype=torch.int64, device="cuda")
        want = torch.zeros(T, dtype=torch.int64, device="cuda")
        call("btb_b200_argmax_bf16", ptr(lg), T, V, ptr(scratch), ptr(want), capi.stream_ptr())
        for _ in range(2):
            got = torch.full((T,), -1, dtype=torch.int64, device="cuda")
            call("btb_b200_argmax_bf16_static", ptr(lg), T, V, ptr(got), capi.stream_ptr())
            torch.cuda.synchronize()
            assert torch.equal(got, want)
            assert int(got[0]) == V // 3
    assert capi.status() == 0


def test_static_scratch_pick_refuses_more_rows_than_it_holds():
    lg = torch.zeros(33, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(33, dtype=torch.int64, device="cuda")
    with pytest.raises(capi.NativeError) as e:
        call("btb_b200_argmax_bf16_static", ptr(lg), 33, 64, ptr(out), capi.stream_ptr())
    assert e.value.rc == capi.ERR_DOMAIN
