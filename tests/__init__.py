"""Tests of dli_b200: CPU tests of the host side and the plain implementation; GPU tests marked ``gpu``."""
