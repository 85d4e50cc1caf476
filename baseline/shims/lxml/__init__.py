"""Stand-in for the absent ``lxml`` package so that the unmodified reference imports.
Only ``lxml.etree`` is used by the reference, and only the ElementTree subset."""
