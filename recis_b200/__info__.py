"""Template-time build information under the reference's module name (``recis/__info__.py:1-5``: an internal-version marker
that the build fills in, and ``is_internal_enabled()`` over it). This build has no proprietary back ends, so the marker is 0;
storage and tracking services plug in at run time instead (``io.table_source``, ``hooks.trace_hook``, ``utils.mos``)."""
INTERVAL_VERSION = "0"


def is_internal_enabled():
    return int(INTERVAL_VERSION)
