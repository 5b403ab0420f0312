"""Tinker-style training API: a request queue with futures in front of one policy worker + engine."""
