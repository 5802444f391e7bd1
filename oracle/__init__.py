"""CPU restatements of the reference's attention path.  Test infrastructure only:
nothing here is imported by the product package."""
