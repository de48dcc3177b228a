"""Test infrastructure only: CPU restatement of the reference's host execution
path.  Nothing under the product package imports this directory."""
