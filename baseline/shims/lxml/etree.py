"""``lxml.etree`` stand-in backed by the standard library (same Element/SubElement/indent/tostring API)."""
from xml.etree.ElementTree import *  # noqa: F401,F403
