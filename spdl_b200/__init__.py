"""B200-native post-decode frame path behind the ``spdl.io`` call surface."""

__version__ = "0.1.0"
