"""``python -m layerstorm_b200.config --emit json-schema|defaults|live-fields|markdown`` / ``--check FILE`` (see ``schema.main``)."""
from .schema import main

raise SystemExit(main())
