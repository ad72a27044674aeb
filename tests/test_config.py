"""CPU: configuration carriers keep the reference's contract (utils/config.py:22-141)."""
import pytest

from packkv_b200.config import PackKVCacheConfig, QuantMethod, QuantMode, RepackMethod


def test_round_trip_equality_and_hash():
    a = PackKVCacheConfig("m", QuantMethod.KIVI, RepackMethod.MEDIAN, False, 64, 192, 16, 0.1, 0.2)
    b = PackKVCacheConfig.from_str(str(a))
    assert a == b and hash(a) == hash(b) and repr(a) == str(a)
    assert b.quant_method.value == (QuantMode.ChannelQuant, QuantMode.TokenQuant)
    c = PackKVCacheConfig("m", QuantMethod.PackKV, RepackMethod.NONE, True, 64, 192, 16, 0.1, 0.2)
    assert a != c and PackKVCacheConfig.from_str(str(c)) == c
    off = PackKVCacheConfig("m", None, None, None, None, None, None, None, None, enable_quant=False)
    assert str(off) == "{'enable_quant': False, 'model_name': 'm'}"
    assert PackKVCacheConfig.from_str(str(off)) == off
    assert a != "not a config"


def test_from_str_does_not_evaluate_code():
    with pytest.raises((ValueError, SyntaxError)):
        PackKVCacheConfig.from_str("__import__('os').system('true')")
