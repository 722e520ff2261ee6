"""Checker code only: see rwkv7_oracle.py.  Never imported by the product package."""
