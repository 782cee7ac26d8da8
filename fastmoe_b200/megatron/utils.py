r"""
Command-line surface of the Megatron adapter.

Parity: ``fmoe/megatron/utils.py:7-20`` — the same six flags with the same defaults, in an
argument group titled ``fastmoe``; newer Megatron-LM versions own ``--num-experts`` themselves,
in which case the expert count is registered as ``--fmoe-num-experts`` instead.
"""
import argparse

# (flag, keyword arguments of ``add_argument``) in the order they appear in ``--help``
_FLAGS = (
    ("--fmoefy", dict(action="store_true", help="turn every transformer MLP into an MoE MLP")),
    ("--num-experts", dict(type=int, default=None, help="experts per GPU")),
    ("--top-k", dict(type=int, default=2, help="experts per token")),
    ("--balance-loss-weight", dict(type=float, default=1, help="weight of the gates' balance loss")),
    ("--balance-strategy", dict(type=str, default=None,
                                help="naive | noisy | gshard | switch | swipe (none: no balance loss)")),
    ("--hidden-hidden-size", dict(type=int, default=None,
                                  help="expert hidden size (default 4 * hidden / top_k / tensor parallel size)")),
)


def add_fmoe_args(parser):
    r"""Register the adapter's flags on ``parser`` (an ``argparse`` parser) and return it."""
    group = parser.add_argument_group(title="fastmoe")
    for flag, kwargs in _FLAGS:
        try:
            group.add_argument(flag, **kwargs)
        except argparse.ArgumentError:
            # only the expert count can collide with a flag Megatron-LM defines itself
            if flag != "--num-experts":
                raise
            group.add_argument("--fmoe-num-experts", **kwargs)
    return parser
