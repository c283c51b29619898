"""Placeholder import path of the layer (fsa/module/fsa.py in the reference); filled in by the
layer implementation."""
