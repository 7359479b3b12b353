"""The role-keyed side-stream pool, with the stream constructor replaced (no GPU needed)."""
from unittest.mock import Mock

import pytest
import torch

from nanoengine_b200.runtime import stream_pool


@pytest.fixture(autouse=True)
def fresh_pool():
    stream_pool.clear_cuda_stream_pool()
    yield
    stream_pool.clear_cuda_stream_pool()


def test_one_stream_per_role_device_and_priority(monkeypatch):
    factory = Mock(side_effect=lambda **kw: object())
    monkeypatch.setattr(torch.cuda, "Stream", factory)
    a = stream_pool.get_cuda_stream("shared_expert", 0)
    assert stream_pool.get_cuda_stream("shared_expert", torch.device("cuda:0")) is a
    assert stream_pool.get_cuda_stream("shared_expert", "cuda:0") is a
    factory.assert_called_once_with(device=0, priority=0)
    others = {stream_pool.get_cuda_stream("draft_chain", 0), stream_pool.get_cuda_stream("shared_expert", 1),
              stream_pool.get_cuda_stream("shared_expert", 0, priority=-1)}
    assert len(others) == 3 and a not in others and factory.call_count == 4
    stream_pool.clear_cuda_stream_pool()
    assert stream_pool.get_cuda_stream("shared_expert", 0) is not a


def test_the_moe_layers_share_the_shared_expert_stream(monkeypatch):
    factory = Mock(side_effect=lambda **kw: object())
    monkeypatch.setattr(torch.cuda, "Stream", factory)
    from nanoengine_b200.models import deepseek
    s0 = deepseek._side_stream(torch.device("cuda:0"))
    assert deepseek._side_stream("cuda:0") is s0 and factory.call_count == 1
