"""CPU restatement of the reference forward. Test infrastructure only: the
product path never imports this package."""
