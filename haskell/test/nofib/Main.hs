{-# LANGUAGE RankNTypes #-}
-- |
-- Module      : nofib-b200
--
-- The reference's property suite (Data.Array.Accelerate.Test.NoFib, built with the
-- @nofib@ flag of package accelerate) run against the B200 backend: the suite takes the
-- backend as a 'RunN' (Test/NoFib/Base.hs:33-34) and compares every result with its list
-- references under 'Similar' (Test/Similar.hs).
--
-- Like the module it tests, this file has never been compiled: it was written where no
-- Haskell toolchain exists.  The same groups are exercised from Python in tests/.
--
-- Half is off in the suite by default (Test/NoFib/Config.hs:65); @--half=True@ turns it on and
-- the backend supports it.  Arguments are handed on to tasty, so a group can be left out by
-- name (@-p '!/simd/'@) while something in it is being worked on.
--
module Main (main) where

import Data.Array.Accelerate.Test.NoFib               ( nofib )
import qualified Data.Array.Accelerate.B200           as B200

import Data.Maybe                                     ( fromMaybe )
import System.Environment                             ( getArgs, lookupEnv, setEnv, withArgs )
import Test.Tasty                                     ( testGroup )

main :: IO ()
main = do
  -- as many cases per property as the interpreter's own driver asks for, unless the caller chose
  cases <- lookupEnv "TASTY_HEDGEHOG_TESTS"
  setEnv "TASTY_HEDGEHOG_TESTS" (fromMaybe "50" cases)
  argv  <- getArgs
  withArgs argv $
    nofib B200.runN (testGroup "runQ" [])     -- no Template Haskell embedding (runQ) for this backend
