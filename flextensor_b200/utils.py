"""Helpers shared by the space, scheduler and drivers.

Mirrors the parts of the reference's ``flextensor/utils.py`` that the hot path uses:
``Config`` (utils.py:11-12), the factor-split enumerators behind ``SplitSpace``
(utils.py:82-128), ``gen_enum`` / ``gen_group`` (utils.py:218-242), ``test_allclose``
(utils.py:267-277) and ``assert_print`` (utils.py:280-282).  The RPC helpers of the
reference (Android boards) have no counterpart here.
"""
import math
from collections import namedtuple

import numpy as np


class Config(namedtuple("Config", ("op_config_lst", "graph_config"))):
    """Result of a search: one knob dict per op plus the graph-level dict.

    ``json.dumps`` turns it into ``[op_config_lst, graph_config]``, the form the drivers
    append to their log and read back with ``Config(obj[0], obj[1])``.
    """


def assert_print(cond, message=""):
    if not cond:
        raise AssertionError(message)


def to_int(expr):
    try:
        return int(expr)
    except Exception as exc:  # same failure type as the reference
        raise RuntimeError("fail to convert to int: %s" % str(exc))


def to_tuple(shape):
    return tuple(to_int(x) for x in shape)


def get_factor_lst(value):
    """Divisors of ``value`` in the reference's order (1, v, 2, v/2, ..., sqrt last)."""
    assert isinstance(value, int) and value > 0
    out = []
    root = math.isqrt(value)
    for i in range(1, root + 1):
        if value % i:
            continue
        j = value // i
        if i == j:
            continue
        out.extend((i, j))
    if root * root == value:
        out.append(root)
    return out


def powerx_lst(x, left, right):
    out, cur = [], 1
    while cur < left:
        cur *= x
    while cur < right:
        out.append(cur)
        cur *= x
    return out


def is_power_of_x(x, val):
    assert isinstance(val, int) and val > 0
    while val % x == 0:
        val //= x
    return val == 1


def any_factor_split(value, number, allow_non_divisible="off"):
    """All ordered ways to write ``value`` as a product of ``number`` parts.

    Policies as in the reference: 'off' uses true divisors, 'power2' also tries powers of
    two (parts then multiply to at least ``value``), 'continuous' tries every integer.
    """
    assert allow_non_divisible in ("off", "power2", "continuous")
    assert_print(isinstance(number, int) and number >= 1)
    out = []

    def rec(left, prefix, parts):
        if parts == 1:
            out.append(prefix + [left])
            return
        if allow_non_divisible == "power2":
            cands = sorted(set(get_factor_lst(left)) | set(powerx_lst(2, 1, left)))
        elif allow_non_divisible == "continuous":
            cands = list(range(1, left + 1))
        else:
            cands = sorted(get_factor_lst(left))
        for f in cands:
            rec(left // f, prefix + [f], parts - 1)

    rec(value, [], number)
    return out


def gen_enum(elements, length):
    """Every length-``length`` sequence over ``elements`` (first element varies slowest)."""
    out = [[]]
    for _ in range(length):
        out = [seq + [e] for seq in out for e in elements]
    return out


def gen_group(elements, most_groups=3):
    """Ways to cut ``elements`` into ``min(len, most_groups)`` contiguous groups.

    A grouping is the list of cut positions; the last position (len) is repeated to pad
    the list to ``most_groups`` entries, as the reference does.
    """
    length = len(elements)
    groups = min(length, most_groups)
    padding = most_groups - groups
    out = []

    def rec(prefix, last, left):
        if left == 1:
            out.append(prefix + [length] * (1 + padding))
            return
        for i in range(last + 1, length):
            rec(prefix + [i], i, left - 1)

    if groups < 1:
        raise RuntimeError("At least 1 group")
    rec([], 0, groups)
    return out


def nearest_power_of_two(val):
    assert isinstance(val, int) and val > 0
    return 1 << (val.bit_length() - 1)


def test_allclose(value, target, rtol=1e-5, print_diff=False):
    """1 if ``value`` matches ``target`` to ``rtol`` (numpy allclose rule, atol 1e-7), else 0."""
    try:
        np.testing.assert_allclose(value, target, rtol=rtol, atol=1e-7)
        return 1
    except AssertionError:
        if print_diff:
            print(target - value)
            print("Max diff:", np.max(np.fabs(target - value)))
        return 0


test_allclose.__test__ = False  # not a pytest test
