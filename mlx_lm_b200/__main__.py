"""``python -m mlx_lm_b200 <subcommand> ...`` as ``mlx_lm <subcommand>`` (mlx_lm/cli.py:7-53)."""
import importlib
import sys

SUBCOMMANDS = {"generate": "mlx_lm_b200.generate", "benchmark": "mlx_lm_b200.benchmark",
               "random_weights": "mlx_lm_b200.weights.loader"}


def main() -> None:
    if len(sys.argv) < 2 or sys.argv[1] in ("-h", "--help"):
        print("usage: python -m mlx_lm_b200 {" + ",".join(SUBCOMMANDS) + "} ...")
        raise SystemExit(0 if len(sys.argv) > 1 else 1)
    if sys.argv[1] == "--version":
        from . import __version__
        print(__version__)
        return
    sub = sys.argv.pop(1)
    if sub not in SUBCOMMANDS:
        raise SystemExit(f"unknown subcommand {sub!r}; choose from {sorted(SUBCOMMANDS)}")
    importlib.import_module(SUBCOMMANDS[sub]).main()


if __name__ == "__main__":
    main()
