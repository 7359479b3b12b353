"""Python entry point of the C++ gateway (``python -m nanoengine_b200.router --port 3001 --ctrl-address ...``).
Parity: reference dlengine/router.py (shim around the Rust `dlengine-router` binary)."""
import sys

from .server.cli import main as _cli_main


def main(argv=None) -> int:
    return _cli_main(["router", *(sys.argv[1:] if argv is None else argv)])


if __name__ == "__main__":
    sys.exit(main())
