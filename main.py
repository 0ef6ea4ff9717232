import sys

from pylon_b200.main import main

__all__ = ["main"]


if __name__ == "__main__":
    sys.exit(main())
