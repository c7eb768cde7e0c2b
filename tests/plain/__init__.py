"""Plain, slow, whole-sequence implementation of the LLaMA decoder used as the
oracle of the test suite.  It has no cache, runs on the CPU in float64 (or any
dtype asked for), has one function per part and shares no code with the
``forge_b200`` package: it even reads safetensors files with its own reader.
"""
