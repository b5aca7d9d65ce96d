"""CPU oracle of the Co-Me hot path (test infrastructure; see ``come_oracle.py`` / ``come_oracle.c``)."""
