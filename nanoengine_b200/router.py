"""Python entry point of the C++ gateway (``python -m nanoengine_b200.router --port 3001 --ctrl-address ...``).
Parity: reference dlengine/router.py (shim around the Rust `dlengine-router` binary)."""
import sys

from .server.cli import main

if __name__ == "__main__":
    sys.exit(main(["router", *sys.argv[1:]]))
