"""``vllm bench serve``: default ``--temperature`` to 0 so benchmark runs are greedy and repeatable.
Parity: vllm_metax/patch/enhancement/chores/bench_serve_args.py:22,284-292."""
from .. import utils


def _install(add_cli_args_orig):
    def add_cli_args(parser):
        add_cli_args_orig(parser)
        for action in getattr(parser, "_actions", []):
            if "--temperature" in getattr(action, "option_strings", ()):
                action.default = 0.0
                return
        try:
            parser.add_argument("--temperature", type=float, default=0.0,
                                help="sampling temperature sent with every benchmark request (default: greedy)")
        except Exception:
            pass

    return add_cli_args


try:
    import vllm.benchmarks.serve as _serve

    if hasattr(_serve, "add_cli_args"):
        utils.apply_patch("vllm.benchmarks.serve", "add_cli_args", _install(_serve.add_cli_args))
except Exception:  # benchmarks extra not installed
    pass
