"""Metaclass that makes a class a process-wide singleton (the role of ``recis/common/singleton.py``).

The one instance is kept on the class itself, creation is guarded by a per-class lock (two threads constructing the first
instance at the same time get the same object), and ``drop_instance()`` forgets it again, which tests use.
"""
from __future__ import annotations

import threading


class SingletonMeta(type):
    def __init__(cls, name, bases, namespace, **kwargs):
        super().__init__(name, bases, namespace, **kwargs)
        cls._the_instance = None
        cls._creation_guard = threading.RLock()

    def __call__(cls, *args, **kwargs):
        found = cls._the_instance
        if found is None:
            with cls._creation_guard:
                found = cls._the_instance
                if found is None:
                    found = cls._the_instance = super().__call__(*args, **kwargs)
        return found

    def drop_instance(cls) -> None:
        with cls._creation_guard:
            cls._the_instance = None
