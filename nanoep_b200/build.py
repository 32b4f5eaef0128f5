"""``python -m nanoep_b200.build``: compile the native extension for this host (alias of utils.build)."""

from .utils.build import main

if __name__ == "__main__":
    main()
