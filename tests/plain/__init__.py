"""A plain, slow implementation of the Qwen3 dense decoder, used only as the oracle of the tests.

It shares no code with ``sleuth_b200``: it has its own safetensors reader, takes whole sequences,
keeps no cache, and has one function per part. Every function cites the file and lines of
tbertha35/Sleuth that give its formula.
"""
