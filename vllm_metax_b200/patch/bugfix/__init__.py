"""Work-arounds for upstream behaviour that is wrong for this platform."""
from . import pp_send_recv  # noqa: F401
