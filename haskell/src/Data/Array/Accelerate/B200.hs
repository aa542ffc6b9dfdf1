{-# LANGUAGE GADTs               #-}
{-# LANGUAGE LambdaCase          #-}
{-# LANGUAGE RankNTypes          #-}
{-# LANGUAGE ScopedTypeVariables #-}
{-# LANGUAGE TypeApplications    #-}
{-# LANGUAGE TypeOperators       #-}
{-# LANGUAGE ForeignFunctionInterface #-}
-- |
-- Module      : Data.Array.Accelerate.B200
-- Description : Execute Accelerate programs on an NVIDIA B200 through libaccb200
--
-- A backend in the sense of "Data.Array.Accelerate.Interpreter": it exports
-- 'run', 'run1' and 'runN' with the interpreter's types (Interpreter.hs:93-126)
-- plus 'runWith' / 'runNWith' taking an explicit handle.  The module is
-- deliberately thin:
--
--   1. the program goes through the stock front end ('convertAcc' /
--      'convertAfun', Trafo.hs:63-85: sharing recovery, let-splitting, fusion);
--   2. the resulting 'DelayedOpenAfun' is written out as program text (one
--      @(let name node)@ per manifest array node, scalar functions as
--      S-expressions) — "Serialise" below;
--   3. the text and the input arrays' payload pointers are handed to the C ABI
--      (include/accelerate_b200.h), which generates, compiles (NVRTC, cached by
--      content hash) and launches the sm_100a kernels;
--   4. results are downloaded into freshly allocated host arrays and wrapped
--      with 'Sugar.toArr'.
--
-- NOTE: no Haskell toolchain was available where this backend was developed, so
-- this module has never been compiled.  Everything below the C ABI is tested
-- (see tests/), and the program-text grammar is exercised by the Python front
-- end; treat this file as the specification of the binding, to be fixed up by
-- the first person who builds it.
--
module Data.Array.Accelerate.B200 (
  B200, createB200, defaultB200,
  run, run1, runN,
  runWith, runNWith,
) where

import Data.Array.Accelerate.AST
import Data.Array.Accelerate.AST.Idx
import Data.Array.Accelerate.AST.LeftHandSide
import Data.Array.Accelerate.AST.Var
import Data.Array.Accelerate.Array.Data                             ( ArrayData, GArrayDataR, ScalarArrayDict(..), scalarArrayDict )
import Data.Array.Accelerate.Representation.Vec                     ( vecRvector )
import Data.Primitive.Vec                                           ( listOfVec )
import Data.Array.Accelerate.Array.Unique                           ( unsafeUniqueArrayPtr, getUniqueId )
import Data.Array.Accelerate.Error
import Data.Array.Accelerate.Representation.Array
import Data.Array.Accelerate.Representation.Shape
import Data.Array.Accelerate.Representation.Stencil
import Data.Array.Accelerate.Representation.Type
import Data.Array.Accelerate.Trafo
import Data.Array.Accelerate.Trafo.Delayed
import Data.Array.Accelerate.Trafo.Sharing                          ( Afunction(..), AfunctionRepr(..), afunctionRepr )
import Data.Array.Accelerate.Type
import qualified Data.Array.Accelerate.Smart                        as Smart
import qualified Data.Array.Accelerate.Sugar.Array                  as Sugar

import Control.Exception                                            ( throwIO, ErrorCall(..), ArithException(..) )
import Control.Monad
import Data.Int
import Data.IORef
import Data.List                                                    ( intercalate )
import Data.Word
import Foreign.C.String
import Foreign.C.Types
import Foreign.Marshal.Alloc
import Foreign.Marshal.Array
import Foreign.Ptr
import Foreign.Storable
import Numeric                                                      ( showHFloat, showHex )
import qualified Data.ByteString                                    as B
import qualified Data.Text                                          as T
import qualified Data.Text.Encoding                                 as T
import System.IO.Unsafe                                             ( unsafePerformIO )


-- C ABI (include/accelerate_b200.h) ------------------------------------------

data Ctx
data Prog

foreign import ccall safe "b200_last_error"     c_lastError    :: IO CString
foreign import ccall safe "b200_ctx_create"     c_ctxCreate    :: CInt -> Word32 -> Ptr (Ptr Ctx) -> IO CInt
foreign import ccall safe "b200_array_new"      c_arrayNew     :: Ptr Ctx -> CString -> CInt -> Ptr Int64 -> Ptr Word64 -> IO CInt
foreign import ccall safe "b200_array_upload"   c_arrayUpload  :: Ptr Ctx -> Word64 -> CInt -> Ptr () -> CSize -> IO CInt
foreign import ccall safe "b200_array_download" c_arrayDownload:: Ptr Ctx -> Word64 -> CInt -> Ptr () -> CSize -> IO CInt
-- copy on a second stream; complete after c_sync
foreign import ccall safe "b200_array_download_async" c_arrayDownloadAsync :: Ptr Ctx -> Word64 -> CInt -> Ptr () -> CSize -> IO CInt
-- lazy variant of c_arrayUpload: the payload is copied when the array is first used; keep it alive
-- (touchArrayData) until the call that uses the array has returned
foreign import ccall safe "b200_array_adopt_host" c_arrayAdoptHost :: Ptr Ctx -> Word64 -> CInt -> Ptr () -> CSize -> IO CInt
foreign import ccall safe "b200_array_free"     c_arrayFree    :: Ptr Ctx -> Word64 -> IO CInt
foreign import ccall safe "b200_array_intern"   c_arrayIntern  :: Ptr Ctx -> Word64 -> CString -> CInt -> Ptr Int64 -> Ptr (Ptr ()) -> Ptr Word64 -> IO CInt
foreign import ccall safe "b200_array_forget"   c_arrayForget  :: Ptr Ctx -> Word64 -> IO CInt
foreign import ccall safe "b200_array_rank"     c_arrayRank    :: Ptr Ctx -> Word64 -> Ptr CInt -> IO CInt
foreign import ccall safe "b200_array_shape"    c_arrayShape   :: Ptr Ctx -> Word64 -> Ptr Int64 -> IO CInt
foreign import ccall safe "b200_program_load"   c_programLoad  :: Ptr Ctx -> CString -> CSize -> Ptr (Ptr Prog) -> IO CInt
foreign import ccall safe "b200_program_run"    c_programRun   :: Ptr Prog -> Ptr Word64 -> CInt -> Ptr Word64 -> CInt -> IO CInt

-- | A backend handle: one GPU, its stream and its kernel cache.
newtype B200 = B200 (Ptr Ctx)

check :: CInt -> IO ()
check 0  = return ()
check rc = do
  msg <- peekCString =<< c_lastError
  -- B200_ERR_BOUNDS (5) corresponds to the reference's boundsCheck failures (Error.hs:52-63);
  -- B200_ERR_ARITH (9) is what GHC raises from quot/rem/div/mod by zero
  if rc == 9 then throwIO DivideByZero
             else throwIO (ErrorCall ("accelerate-b200 [" ++ show rc ++ "]: " ++ msg))

-- | Open a context on the given CUDA device.
createB200 :: Int -> IO B200
createB200 dev = alloca $ \p -> do
  check =<< c_ctxCreate (fromIntegral dev) 0 p
  B200 <$> peek p

{-# NOINLINE defaultB200 #-}
defaultB200 :: B200
defaultB200 = unsafePerformIO (createB200 0)


-- Front door (Interpreter.hs:93-126) ------------------------------------------

run :: Sugar.Arrays a => Smart.Acc a -> a
run = runWith defaultB200

runWith :: forall a. Sugar.Arrays a => B200 -> Smart.Acc a -> a
runWith h a = unsafePerformIO $ do
  let acc  = convertAcc a                       -- DelayedAcc (ArraysR a)
      afun = Abody acc
  prog <- loadProgram h afun
  Sugar.toArr <$> execute h prog (arraysR acc) []

run1 :: (Sugar.Arrays a, Sugar.Arrays b) => (Smart.Acc a -> Smart.Acc b) -> a -> b
run1 = runN

runN :: forall f. Afunction f => f -> AfunctionR f
runN = runNWith defaultB200

-- | The program is converted, serialised and loaded once; each application
-- of the result only uploads, runs and downloads.
runNWith :: forall f. Afunction f => B200 -> f -> AfunctionR f
runNWith h f = go
  where
    !afun = convertAfun f
    !prog = unsafePerformIO (loadProgram h afun)
    !go   = eval (afunctionRepr @f) afun []

    eval :: AfunctionRepr g (AfunctionR g) (ArraysFunctionR g)
         -> DelayedOpenAfun aenv (ArraysFunctionR g)
         -> [HostArrays]
         -> AfunctionR g
    eval (AfunctionReprLam repr) (Alam lhs body) args = \x ->
      eval repr body (args ++ [HostArrays (lhsToTupR lhs) (Sugar.fromArr x)])
    eval AfunctionReprBody (Abody b) args = unsafePerformIO $
      Sugar.toArr <$> execute h prog (arraysR b) args
    eval _ _ _ = error "runN: function/body mismatch"

data HostArrays = forall a. HostArrays (ArraysR a) a

newtype Program = Program (Ptr Prog)

loadProgram :: B200 -> DelayedOpenAfun () f -> IO Program
loadProgram (B200 ctx) afun =
  withCStringLen (serialiseAfun afun) $ \(p, n) -> alloca $ \out -> do
    check =<< c_programLoad ctx p (fromIntegral n) out
    Program <$> peek out

-- | Upload the arguments (one device array per input 'Array', one leaf per
-- scalar component of the element type, Array/Data.hs:95-98), run, and download
-- every result into a fresh host array ('allocateArray', Representation/Array.hs:94-97).
execute :: B200 -> Program -> ArraysR r -> [HostArrays] -> IO r
execute (B200 ctx) (Program prog) resR args = do
  ins  <- concat <$> mapM (\(HostArrays r a) -> uploadArrays ctx r a) args
  let nout = countArrays resR
  outs <- withArrayLen ins $ \nin pin -> allocaArray nout $ \pout -> do
    check =<< c_programRun prog pin (fromIntegral nin) pout (fromIntegral nout)
    peekArray nout pout
  mapM_ (c_arrayFree ctx) ins
  ref <- newIORef outs
  downloadArrays ctx resR ref

countArrays :: ArraysR a -> Int
countArrays TupRunit       = 0
countArrays (TupRsingle _) = 1
countArrays (TupRpair a b) = countArrays a + countArrays b

uploadArrays :: Ptr Ctx -> ArraysR a -> a -> IO [Word64]
uploadArrays _   TupRunit         ()     = return []
uploadArrays ctx (TupRpair ra rb) (a, b) = (++) <$> uploadArrays ctx ra a <*> uploadArrays ctx rb b
uploadArrays ctx (TupRsingle (ArrayR shr tp)) (Array sh adata) = do
  let dims = map fromIntegral (shapeToList shr sh) :: [Int64]
      n    = size shr sh
  -- The device copy is keyed by the unique id of the array's first leaf (Array/Unique.hs:48-51), as in
  -- the reference's memory table (Array/Remote/Table.hs:89-100): an array passed to several runs is
  -- uploaded once.  (A finalizer on the array calls b200_array_forget: Array/Remote/Table.hs:271-284.)
  ptrs <- newIORef []
  _ <- forLeaves tp adata 0 $ \_ _ ptr -> modifyIORef ptrs (ptr :)
  leaves <- reverse <$> readIORef ptrs
  let _ = n
  let (eltText, dims') = case vectorElt tp of
        Just (w, t) -> (t, fromIntegral w : dims)       -- innermost first, like shapeToList
        Nothing     -> (typeText tp, dims)
  ident <- withCString eltText $ \ty -> withArrayLen (reverse dims') $ \r pd ->
           withArray leaves $ \pl -> alloca $ \pid -> do
    check =<< c_arrayIntern ctx (arrayKey tp adata) ty (fromIntegral r) pd pl pid      -- shapeToList is innermost-first
    peek pid
  return [ident]

downloadArrays :: Ptr Ctx -> ArraysR a -> IORef [Word64] -> IO a
downloadArrays _   TupRunit         _   = return ()
downloadArrays ctx (TupRpair ra rb) ref = (,) <$> downloadArrays ctx ra ref <*> downloadArrays ctx rb ref
downloadArrays ctx (TupRsingle repr@(ArrayR shr tp)) ref = do
  ident <- atomicModifyIORef' ref (\(x:xs) -> (xs, x))
  rank  <- alloca $ \p -> c_arrayRank ctx ident p >>= check >> fromIntegral <$> peek p
  dims  <- allocaArray (max 1 rank) $ \p -> c_arrayShape ctx ident p >>= check >> peekArray rank p
  let outer = maybe id (const init) (vectorElt tp)        -- the components' dimension is no part of the shape
      sh    = listToShape shr (reverse (map fromIntegral (outer (dims :: [Int64]))))
  arr@(Array _ adata) <- allocateArray repr sh
  forLeaves tp adata 0 $ \leaf bytesPer ptr ->
    check =<< c_arrayDownload ctx ident (fromIntegral leaf) ptr (fromIntegral (size shr sh * bytesPer))
  _ <- c_arrayFree ctx ident
  return arr

-- | Key of an array in the memory table: the unique id of its first scalar leaf (every leaf of a
-- struct-of-arrays payload is allocated together and dies together).
arrayKey :: TypeR e -> ArrayData e -> Word64
arrayKey TupRunit        ()     = 0
arrayKey (TupRpair ta _) (a, _) = arrayKey ta a
arrayKey (TupRsingle t)  ad     = fromIntegral (unsafePerformIO (scalarUniqueId t ad))

-- | Visit the payload pointer of every scalar leaf, left to right.
forLeaves :: TypeR e -> ArrayData e -> Int -> (Int -> Int -> Ptr () -> IO ()) -> IO Int
forLeaves TupRunit         ()       k _ = return k
forLeaves (TupRpair ta tb) (a, b)   k f = forLeaves ta a k f >>= \k' -> forLeaves tb b k' f
forLeaves (TupRsingle t)   ad       k f = do
  let (bytesPer, ptr) = scalarPayload t ad
  f k bytesPer ptr
  return (k + 1)

-- Pointer to the pinned host payload of one scalar leaf ('unsafeUniqueArrayPtr').
scalarPayload :: ScalarType t -> ArrayData t -> (Int, Ptr ())
scalarPayload (SingleScalarType (NumSingleType nt)) ad = case nt of
  IntegralNumType it -> case it of
    TypeInt    -> (8, castPtr (unsafeUniqueArrayPtr ad)); TypeInt8   -> (1, castPtr (unsafeUniqueArrayPtr ad))
    TypeInt16  -> (2, castPtr (unsafeUniqueArrayPtr ad)); TypeInt32  -> (4, castPtr (unsafeUniqueArrayPtr ad))
    TypeInt64  -> (8, castPtr (unsafeUniqueArrayPtr ad)); TypeWord   -> (8, castPtr (unsafeUniqueArrayPtr ad))
    TypeWord8  -> (1, castPtr (unsafeUniqueArrayPtr ad)); TypeWord16 -> (2, castPtr (unsafeUniqueArrayPtr ad))
    TypeWord32 -> (4, castPtr (unsafeUniqueArrayPtr ad)); TypeWord64 -> (8, castPtr (unsafeUniqueArrayPtr ad))
  FloatingNumType ft -> case ft of
    TypeFloat  -> (4, castPtr (unsafeUniqueArrayPtr ad)); TypeDouble -> (8, castPtr (unsafeUniqueArrayPtr ad))
    TypeHalf   -> (2, castPtr (unsafeUniqueArrayPtr ad))   -- the 16 bits of Numeric.Half, as the library keeps them
-- An array of @Vec n t@ is one payload of t, n per element (Array/Data.hs:108-119): n * sizeof t bytes each.
scalarPayload t@(VectorScalarType (VectorType w s)) ad
  | ScalarArrayDict _ _ <- scalarArrayDict t = (w * singleBytes s, castPtr (unsafeUniqueArrayPtr ad))

-- 'getUniqueId' of the leaf's 'UniqueArray' (Array/Unique.hs:48-51, 66-69).
scalarUniqueId :: ScalarType t -> ArrayData t -> IO Int
scalarUniqueId (SingleScalarType (NumSingleType nt)) ad = case nt of
  IntegralNumType it -> case it of
    TypeInt    -> getUniqueId ad; TypeInt8   -> getUniqueId ad; TypeInt16  -> getUniqueId ad; TypeInt32  -> getUniqueId ad
    TypeInt64  -> getUniqueId ad; TypeWord   -> getUniqueId ad; TypeWord8  -> getUniqueId ad; TypeWord16 -> getUniqueId ad
    TypeWord32 -> getUniqueId ad; TypeWord64 -> getUniqueId ad
  FloatingNumType ft -> case ft of
    TypeFloat  -> getUniqueId ad; TypeDouble -> getUniqueId ad
    TypeHalf   -> getUniqueId ad
scalarUniqueId t@VectorScalarType{} ad
  | ScalarArrayDict _ _ <- scalarArrayDict t = getUniqueId ad

singleBytes :: SingleType t -> Int
singleBytes (NumSingleType nt) = case nt of
  IntegralNumType it -> case it of
    TypeInt -> 8; TypeInt8 -> 1; TypeInt16 -> 2; TypeInt32 -> 4; TypeInt64 -> 8
    TypeWord -> 8; TypeWord8 -> 1; TypeWord16 -> 2; TypeWord32 -> 4; TypeWord64 -> 8
  FloatingNumType ft -> case ft of
    TypeHalf -> 2; TypeFloat -> 4; TypeDouble -> 8

-- | @Just (n, t)@ when the elements of an array are SIMD vectors.  Such an array goes to the library as
-- an array of t with one more, innermost, dimension of extent n: the same bytes.  (Vectors inside a
-- tuple element have no such reading and are refused.)
vectorElt :: TypeR e -> Maybe (Int, String)
vectorElt (TupRsingle (VectorScalarType (VectorType w s))) = Just (w, scalarText (SingleScalarType s))
vectorElt _                                                = Nothing

unsupported :: String -> a
unsupported what = error ("accelerate-b200: " ++ what ++ " are not supported by this backend")


-- Serialise --------------------------------------------------------------------
--
-- Program text grammar (accepted by b200_program_load):
--
--   program := (program (in NAME (array RANK ELT))* (let LHS NODE)* (out NAME+))
--   NODE    := (generate ELT sh fun) | (fold ELT fun [seed] D) | (foldseg ELT fun [seed] D Dseg)
--            | (scanl|scanr ELT fun [seed] D) | (scanl'|scanr' ELT fun seed D)
--            | (permute ELT fun DEFAULTS ixfun D) | (stencil ELT stencilr fun bnd D)
--            | (stencil2 ELT stencilr stencilr fun bnd D bnd D) | (reshape sh NAME)
--            | (use (array RANK ELT) (shape d..) (hex BYTES)+)        -- Use: one (hex ..) per scalar leaf
--            | (acond exp (branch BODY) (branch BODY))                 -- Acond
--            | (awhile AFUN AFUN (args NAME*)) | (apply AFUN (args NAME*))
--            | (atrace (hex MESSAGE) (show NAME*) (args NAME*))        -- Atrace: print, then hand the args on
--   AFUN    := (afun ((NAME (array RANK ELT))*) BODY)
--   BODY    := (let LHS NODE)* (out NAME+)
--   D       := (manifest NAME) | (delayed extent fun)
--
-- Tuples are the representation's snoc lists: Nil = (tup), Pair l r = (snoc l r).

data Names aenv = Names { arrayName :: forall t. Idx aenv t -> String }

emptyNames :: Names ()
emptyNames = Names (\_ -> error "unbound array variable")

-- State threaded through serialisation: fresh-name counter and emitted lines.
data S = S { fresh :: !Int, inputs :: [String], lets :: [String] }

serialiseAfun :: DelayedOpenAfun () f -> String
serialiseAfun afun =
  let (outs, s) = goFun afun emptyNames (S 0 [] [])
  in  unlines (["(program"] ++ reverse (inputs s) ++ reverse (lets s) ++ ["  (out " ++ unwords outs ++ "))"])
  where
    goFun :: DelayedOpenAfun aenv g -> Names aenv -> S -> ([String], S)
    goFun (Abody b)    ns s = manifestArrays b ns s
    goFun (Alam lhs f) ns s =
      let (ns', s') = bindInputs lhs ns s in goFun f ns' s'

-- Parameters of the function become (in ...) declarations.
bindInputs :: ALeftHandSide a aenv aenv' -> Names aenv -> S -> (Names aenv', S)
bindInputs (LeftHandSideWildcard _) ns s = (ns, s)
bindInputs (LeftHandSidePair a b)   ns s = let (ns', s') = bindInputs a ns s in bindInputs b ns' s'
bindInputs (LeftHandSideSingle (ArrayR shr tp)) ns s =
  let nm = "a" ++ show (fresh s)
      d  = "  (in " ++ nm ++ " (array " ++ show (rank shr) ++ " " ++ typeText tp ++ "))"
  in  (push ns nm, s { fresh = fresh s + 1, inputs = d : inputs s })

push :: Names aenv -> String -> Names (aenv, t)
push (Names f) nm = Names (\case ZeroIdx -> nm; SuccIdx i -> f i)

-- Evaluate an array term to the names of the manifest arrays it denotes.
manifestArrays :: DelayedOpenAcc aenv a -> Names aenv -> S -> ([String], S)
manifestArrays (Manifest pacc) ns s = case pacc of
  Avar (Var _ ix)   -> ([arrayName ns ix], s)
  Anil              -> ([], s)
  Apair a b         -> let (xs, s1) = manifestArrays a ns s; (ys, s2) = manifestArrays b ns s1 in (xs ++ ys, s2)
  Alet lhs bnd body -> let (xs, s1)  = manifestArrays bnd ns s
                           ns'       = bindNames lhs xs ns
                       in  manifestArrays body ns' s1
  _                 -> emitNode pacc ns s
manifestArrays Delayed{} _ _ = internalError "delayed array in manifest position (Fusion.hs:161-216 rules this out)"

bindNames :: ALeftHandSide a aenv aenv' -> [String] -> Names aenv -> Names aenv'
bindNames lhs xs ns = fst (go lhs xs ns)
  where
    go :: ALeftHandSide b e e' -> [String] -> Names e -> (Names e', [String])
    go (LeftHandSideWildcard r) ys n = (n, drop (countArrays r) ys)
    go (LeftHandSideSingle _)   (y:ys) n = (push n y, ys)
    go (LeftHandSideSingle _)   []     _ = internalError "array binding without a value"
    go (LeftHandSidePair a b)   ys n = let (n', ys') = go a ys n in go b ys' n'

-- One executable node = one (let ...) line.
emitNode :: PreOpenAcc DelayedOpenAcc aenv a -> Names aenv -> S -> ([String], S)
emitNode pacc ns s0 =
  let nouts       = case pacc of
                      Scan'{}  -> 2
                      Acond{}  -> countArrays (arraysR pacc)
                      Awhile{} -> countArrays (arraysR pacc)
                      Apply{}  -> countArrays (arraysR pacc)
                      _        -> 1
      names       = [ "a" ++ show (fresh s0 + k) | k <- [0 .. nouts - 1] ]
      s1          = s0 { fresh = fresh s0 + nouts }
      (body, s2)  = nodeText pacc ns s1
      lhs         = case names of [n] -> n; _ -> "(" ++ unwords names ++ ")"
  in  (names, s2 { lets = ("  (let " ++ lhs ++ " " ++ body ++ ")") : lets s2 })

nodeText :: PreOpenAcc DelayedOpenAcc aenv a -> Names aenv -> S -> (String, S)
nodeText pacc ns s = case pacc of
  Use (ArrayR shr tp) (Array sh adata)
                               -> let dims = reverse (shapeToList shr sh)          -- shapeToList is innermost-first
                                  in  (sx (["use", "(array " ++ show (rank shr) ++ " " ++ typeText tp ++ ")", sx ("shape" : map show dims)]
                                           ++ hexLeaves tp adata (size shr sh)), s)
  Unit tp e                    -> (sx ["generate", typeText tp, "(tup)", lam1 "(tup)" (\_ -> expText ns [] e)], s)
  Generate (ArrayR _ tp) sh f  -> (sx ["generate", typeText tp, expText ns [] sh, funText ns f], s)
  Map tp f a                   -> let (d, s') = operand a ns s
                                  in  (sx ["generate", typeText tp, extentOf d, composeText ns (arrayRshape (arrayR a)) f d], s')
  Backpermute shr sh p a       -> let (d, s') = operand a ns s
                                  in  (sx ["generate", typeText (arrayRtype (arrayR a)), expText ns [] sh, backpermuteText ns shr p d], s')
  Transform (ArrayR shr tp) sh p f a
                               -> let (d, s') = operand a ns s
                                  in  (sx ["generate", typeText tp, expText ns [] sh, transformText ns shr p f d], s')
  Reshape _ sh a               -> let ([n], s') = manifestArrays a ns s in (sx ["reshape", expText ns [] sh, n], s')
  Fold f z a                   -> let (d, s') = operand a ns s
                                  in  (sx (["fold", eltOf a, funText ns f] ++ seed z ++ [operandText d]), s')
  FoldSeg _ f z a seg          -> let (d, s1) = operand a ns s; (g, s2) = operand seg ns s1
                                  in  (sx (["foldseg", eltOf a, funText ns f] ++ seed z ++ [operandText d, operandText g]), s2)
  Scan dir f z a               -> let (d, s') = operand a ns s
                                  in  (sx ([scanName dir False, eltOf a, funText ns f] ++ seed z ++ [operandText d]), s')
  Scan' dir f z a              -> let (d, s') = operand a ns s
                                  in  (sx [scanName dir True, eltOf a, funText ns f, expText ns [] z, operandText d], s')
  Permute f def p a            -> let ([dn], s1) = manifestArrays def ns s; (d, s2) = operand a ns s1
                                  in  (sx ["permute", eltOf a, funText ns f, dn, funText ns p, operandText d], s2)
  Stencil sr tp f b a          -> let (d, s') = operand a ns s
                                  in  (sx ["stencil", typeText tp, stencilText sr, funText ns f, boundaryText ns (arrayR a) b, operandText d], s')
  Stencil2 s1r s2r tp f b1 a1 b2 a2
                               -> let (d1, sa) = operand a1 ns s; (d2, sb) = operand a2 ns sa
                                  in  (sx ["stencil2", typeText tp, stencilText s1r, stencilText s2r, funText ns f,
                                           boundaryText ns (arrayR a1) b1, operandText d1, boundaryText ns (arrayR a2) b2, operandText d2], sb)
  -- evaluated on the host by the library, as by every backend (Interpreter.hs:215-229)
  Acond p t e                  -> let (tb, s1) = subBody "branch" (manifestArrays t ns) s
                                      (eb, s2) = subBody "branch" (manifestArrays e ns) s1
                                  in  (sx ["acond", expText ns [] p, tb, eb], s2)
  Awhile c f a                 -> let (xs, s1) = manifestArrays a ns s
                                      (cb, s2) = afunText c ns s1
                                      (fb, s3) = afunText f ns s2
                                  in  (sx ["awhile", cb, fb, sx ("args" : xs)], s3)
  Apply _ f a                  -> let (xs, s1) = manifestArrays a ns s
                                      (fb, s2) = afunText f ns s1
                                  in  (sx ["apply", fb, sx ("args" : xs)], s2)
  -- no foreign implementation is registered for this backend: the pure fallback runs, as in the
  -- interpreter (Interpreter.hs:217)
  Aforeign _ _ f a             -> let (xs, s1) = manifestArrays a ns s
                                      (fb, s2) = afunText f ns s1
                                  in  (sx ["apply", fb, sx ("args" : xs)], s2)
  -- Interpreter.hs:215: the library prints the message and its own rendering of the arrays (the
  -- Message's `show` is a Haskell closure and stays on this side of the boundary)
  Atrace (Message _ _ msg) a b -> let (xs, s1) = manifestArrays a ns s
                                      (ys, s2) = manifestArrays b ns s1
                                  in  (sx ["atrace", sx ["hex", hexText msg], sx ("show" : xs), sx ("args" : ys)], s2)
  _                            -> internalError "node should have been fused away (Fusion.hs:198-200)"
  where
    seed Nothing  = []
    seed (Just z) = [expText ns [] z]
    eltOf a = typeText (arrayRtype (arrayR a))
    scanName LeftToRight p = if p then "scanl'" else "scanl"
    scanName RightToLeft p = if p then "scanr'" else "scanr"

-- The nodes of a branch or of an array-level function, serialised on their own and wrapped.
subBody :: String -> (S -> ([String], S)) -> S -> (String, S)
subBody hd k s =
  let (outs, s') = k s { lets = [] }
  in  ("(" ++ hd ++ " " ++ unwords (reverse (lets s')) ++ " (out " ++ unwords outs ++ "))", s' { lets = lets s })

-- (afun ((p (array R T)) ...) (let ..)* (out ..)) for a unary array-level function
afunText :: DelayedOpenAfun aenv f -> Names aenv -> S -> (String, S)
afunText (Alam lhs (Abody b)) ns s =
  let (ns', ps, s1) = bindParams lhs ns s
  in  subBody ("afun (" ++ unwords ps ++ ")") (manifestArrays b ns') s1
afunText _ _ _ = internalError "array-level function of unexpected arity"

bindParams :: ALeftHandSide a aenv aenv' -> Names aenv -> S -> (Names aenv', [String], S)
bindParams (LeftHandSideWildcard _) ns s = (ns, [], s)
bindParams (LeftHandSidePair a b)   ns s =
  let (ns1, p1, s1) = bindParams a ns s; (ns2, p2, s2) = bindParams b ns1 s1 in (ns2, p1 ++ p2, s2)
bindParams (LeftHandSideSingle (ArrayR shr tp)) ns s =
  let nm = "a" ++ show (fresh s)
  in  (push ns nm, ["(" ++ nm ++ " (array " ++ show (rank shr) ++ " " ++ typeText tp ++ "))"], s { fresh = fresh s + 1 })

-- Payload of an embedded array: the bytes of every scalar leaf as hexadecimal text.
-- UTF-8 bytes of a message as hex digits
hexText :: T.Text -> String
hexText = concatMap byte . B.unpack . T.encodeUtf8
  where byte w = let h = showHex w "" in if length h == 1 then '0' : h else h

hexLeaves :: TypeR e -> ArrayData e -> Int -> [String]
hexLeaves tp ad n = unsafePerformIO $ do
  ref <- newIORef []
  _ <- forLeaves tp ad 0 $ \_ bytesPer ptr -> do
         bytes <- peekArray (n * bytesPer) (castPtr ptr :: Ptr Word8)
         modifyIORef ref (("(hex " ++ concatMap (\b -> showHex2 b) bytes ++ ")") :)
  reverse <$> readIORef ref
  where
    showHex2 b = let h = showHex b "" in if length h == 1 then '0' : h else h

-- An operand is either a manifest array (by name) or a delayed array.
data Operand = OManifest String Int | ODelayed String String     -- extent text, index function text

operand :: DelayedOpenAcc aenv (Array sh e) -> Names aenv -> S -> (Operand, S)
operand (Delayed _ sh f _) ns s = (ODelayed (expText ns [] sh) (funText ns f), s)
operand m@(Manifest _)     ns s = let ([n], s') = manifestArrays m ns s
                                  in  (OManifest n (rank (arrayRshape (arrayR m))), s')

operandText :: Operand -> String
operandText (OManifest n _)  = sx ["manifest", n]
operandText (ODelayed sh f)  = sx ["delayed", sh, f]

extentOf :: Operand -> String
extentOf (OManifest n _) = sx ["shape", n]
extentOf (ODelayed sh _) = sh

indexOperand :: Operand -> String -> String
indexOperand (OManifest n _) ix = sx ["index", n, ix]
indexOperand (ODelayed _ f)  ix = sx ["app", f, ix]

shapeTypeText :: ShapeR sh -> String
shapeTypeText shr = sx ("tup" : replicate (rank shr) "i64")

-- \ix -> f (a ! ix)
composeText :: Names aenv -> ShapeR sh -> Fun aenv (a -> b) -> Operand -> String
composeText ns shr f d = lamT (shapeTypeText shr) (\ix -> sx ["app", funText ns f, indexOperand d ix])

backpermuteText :: Names aenv -> ShapeR sh' -> Fun aenv (sh' -> sh) -> Operand -> String
backpermuteText ns shr p d = lamT (shapeTypeText shr) (\ix -> indexOperand d (sx ["app", funText ns p, ix]))

transformText :: Names aenv -> ShapeR sh' -> Fun aenv (sh' -> sh) -> Fun aenv (a -> b) -> Operand -> String
transformText ns shr p f d = lamT (shapeTypeText shr) (\ix -> sx ["app", funText ns f, indexOperand d (sx ["app", funText ns p, ix])])

lam1 :: String -> (String -> String) -> String
lam1 = lamT

lamT :: String -> (String -> String) -> String
lamT ty body = "(lam ((%ix " ++ ty ++ ")) " ++ body "(var %ix)" ++ ")"

stencilText :: StencilR sh e pat -> String
stencilText sr = sx ("stencilr" : map show (extents sr))
  where
    extents :: StencilR sh e pat -> [Int]
    extents StencilRunit3{} = [3]
    extents StencilRunit5{} = [5]
    extents StencilRunit7{} = [7]
    extents StencilRunit9{} = [9]
    extents (StencilRtup3 a _ _)             = 3 : extents a
    extents (StencilRtup5 a _ _ _ _)         = 5 : extents a
    extents (StencilRtup7 a _ _ _ _ _ _)     = 7 : extents a
    extents (StencilRtup9 a _ _ _ _ _ _ _ _) = 9 : extents a

boundaryText :: Names aenv -> ArrayR (Array sh e) -> Boundary aenv (Array sh e) -> String
boundaryText _  _ Clamp        = "clamp"
boundaryText _  _ Mirror       = "mirror"
boundaryText _  _ Wrap         = "wrap"
boundaryText _  (ArrayR _ tp) (Constant v) = sx ["constant", constText tp v]
boundaryText ns _ (Function f) = sx ["function", funText ns f]

-- Scalar functions and expressions ----------------------------------------------
-- Scalar variables are named by their de Bruijn level.

funText :: Names aenv -> Fun aenv f -> String
funText ns = openFunText ns []

openFunText :: Names aenv -> [String] -> OpenFun env aenv f -> String
openFunText ns env fun = "(lam (" ++ unwords params ++ ") " ++ body ++ ")"
  where
    (params, body) = go (length env) env fun
    go :: Int -> [String] -> OpenFun env' aenv f' -> ([String], String)
    go _ e (Body b)    = ([], openExpText ns e b)
    go k e (Lam lhs f) =
      let p          = "p" ++ show k
          (e', wrap) = bindScalars lhs ("(var " ++ p ++ ")") e
          (ps, b)    = go (k + 1 + lhsSize lhs) e' f
      in  (("(" ++ p ++ " " ++ typeText (lhsToTupR lhs) ++ ")") : ps, wrap b)

lhsSize :: LeftHandSide s v env env' -> Int
lhsSize LeftHandSideSingle{}   = 1
lhsSize LeftHandSideWildcard{} = 0
lhsSize (LeftHandSidePair a b) = lhsSize a + lhsSize b

-- Bind the scalar variables of a pattern to components of `val`; returns the new
-- environment (innermost variable first) and a wrapper introducing the lets.
bindScalars :: ELeftHandSide t env env' -> String -> [String] -> ([String], String -> String)
bindScalars LeftHandSideWildcard{} _   env = (env, id)
bindScalars LeftHandSideSingle{}   val env =
  let v = "x" ++ show (length env) in (v : env, \b -> sx ["let", v, val, b])
bindScalars (LeftHandSidePair l r) val env =
  let (env1, w1) = bindScalars l (sx ["init", val]) env
      (env2, w2) = bindScalars r (lastOf val) env1
  in  (env2, w1 . w2)
  where lastOf v = sx ["last", v]     -- (last v): the final component of a snoc tuple

expText :: Names aenv -> [String] -> OpenExp env aenv t -> String
expText = openExpText

openExpText :: forall env aenv t. Names aenv -> [String] -> OpenExp env aenv t -> String
openExpText ns env = go
  where
    go :: OpenExp env aenv s -> String
    go = \case
      Let lhs a b         -> let (env', wrap) = bindScalars lhs (go a) env in wrap (openExpText ns env' b)
      Evar (Var _ ix)     -> sx ["var", env !! idxToInt ix]
      Pair a b            -> sx ["snoc", goL a, go b]
      Nil                 -> "(tup)"
      Const t c           -> constText (TupRsingle t) c
      Undef t             -> sx ["undef", scalarText t]
      PrimConst c         -> primConstText c
      PrimApp f x         -> primText f (go x)
      Cond c t e          -> sx ["cond", go c, go t, go e]
      Case e rhs def      -> sx (["case", go e, "(" ++ unwords [ "(" ++ show tag ++ " " ++ go r ++ ")" | (tag, r) <- rhs ] ++ ")"]
                                 ++ maybe [] (\d -> [go d]) def)
      While p f x         -> sx ["while", openFunText ns env p, openFunText ns env f, go x]
      Index (Var _ a) ix  -> sx ["index", arrayName ns a, go ix]
      LinearIndex (Var _ a) i -> sx ["lindex", arrayName ns a, go i]
      Shape (Var _ a)     -> sx ["shape", arrayName ns a]
      ShapeSize _ sh      -> sx ["shapesize", go sh]
      ToIndex _ sh ix     -> sx ["toindex", go sh, go ix]
      FromIndex _ sh i    -> sx ["fromindex", go sh, go i]
      Coerce t1 t2 e      -> sx ["coerce", scalarText t1, scalarText t2, go e]
      Foreign{}           -> unsupported "foreign scalar functions"
      VecPack vecR e      | VectorType w s <- vecRvector vecR
                          -> sx ["vecpack",   show w, scalarText (SingleScalarType s), go e]
      VecUnpack vecR e    | VectorType w s <- vecRvector vecR
                          -> sx ["vecunpack", show w, scalarText (SingleScalarType s), go e]
      IndexSlice{}        -> unsupported "IndexSlice (use the fused Transform form)"
      IndexFull{}         -> unsupported "IndexFull (use the fused Transform form)"
    goL :: OpenExp env aenv s -> String
    goL = go

sx :: [String] -> String
sx xs = "(" ++ unwords xs ++ ")"

-- Types -------------------------------------------------------------------------

typeText :: TypeR t -> String
typeText TupRunit       = "(tup)"
typeText (TupRsingle t) = scalarText t
typeText t@TupRpair{}   = sx ("tup" : components t)
  where
    -- snoc list: (((), a), b) has components [a, b]
    components :: TypeR s -> [String]
    components TupRunit       = []
    components (TupRpair l r) = components l ++ [typeText r]
    components s              = [typeText s]

scalarText :: ScalarType t -> String
scalarText (SingleScalarType (NumSingleType nt)) = case nt of
  IntegralNumType it -> case it of
    TypeInt -> "i64"; TypeInt8 -> "i8"; TypeInt16 -> "i16"; TypeInt32 -> "i32"; TypeInt64 -> "i64"
    TypeWord -> "u64"; TypeWord8 -> "u8"; TypeWord16 -> "u16"; TypeWord32 -> "u32"; TypeWord64 -> "u64"
  FloatingNumType ft -> case ft of
    TypeFloat -> "f32"; TypeDouble -> "f64"; TypeHalf -> "f16"
scalarText (VectorScalarType (VectorType w s)) = sx ["vec", show w, scalarText (SingleScalarType s)]

constText :: TypeR t -> t -> String
constText TupRunit         ()     = "(tup)"
constText (TupRpair ta tb) (a, b) = sx ["snoc", constText ta a, constText tb b]
-- a constant vector is the pack of its constant components (as 'showElt' takes it apart, Representation/Elt.hs:150-154)
constText (TupRsingle (VectorScalarType (VectorType w s))) v
  | SingleDict <- singleDict s
  , st         <- scalarText (SingleScalarType s)
  = sx ["vecpack", show w, st, sx ("tup" : [ sx ["const", st, literal (SingleScalarType s) x] | x <- listOfVec v ])]
constText (TupRsingle t)   v      = sx ["const", scalarText t, literal t v]

-- Integers in decimal; floating point as C99 hexadecimal literals (exact).
literal :: ScalarType t -> t -> String
literal (SingleScalarType (NumSingleType nt)) v = case nt of
  IntegralNumType it | IntegralDict <- integralDict it -> show (toInteger v)
  FloatingNumType ft -> case ft of
    TypeFloat  -> hex (realToFrac v :: Double)
    TypeDouble -> hex v
    TypeHalf   -> hex (realToFrac v :: Double)   -- exact: every Half is a Double
  where hex d | isNaN d = "nan" | isInfinite d = if d > 0 then "inf" else "-inf" | otherwise = showHFloat d ""
literal VectorScalarType{} _ = unsupported "SIMD vector constants outside constText"

primConstText :: PrimConst t -> String
primConstText (PrimMinBound (IntegralBoundedType t)) = sx ["minbound", scalarText (SingleScalarType (NumSingleType (IntegralNumType t)))]
primConstText (PrimMaxBound (IntegralBoundedType t)) = sx ["maxbound", scalarText (SingleScalarType (NumSingleType (IntegralNumType t)))]
primConstText (PrimPi t)                             = sx ["pi", scalarText (SingleScalarType (NumSingleType (FloatingNumType t)))]

-- Primitive application: (prim NAME TYPE [TYPE2] ARG); a binary primitive receives its
-- arguments as one pair, which the C side accepts as such (AST.hs:560).
primText :: PrimFun (a -> r) -> String -> String
primText f x = case f of
  PrimAdd t -> n "add" (num t); PrimSub t -> n "sub" (num t); PrimMul t -> n "mul" (num t)
  PrimNeg t -> n "neg" (num t); PrimAbs t -> n "abs" (num t); PrimSig t -> n "sig" (num t)
  PrimQuot t -> n "quot" (int t); PrimRem t -> n "rem" (int t); PrimQuotRem t -> n "quotrem" (int t)
  PrimIDiv t -> n "idiv" (int t); PrimMod t -> n "mod" (int t); PrimDivMod t -> n "divmod" (int t)
  PrimBAnd t -> n "band" (int t); PrimBOr t -> n "bor" (int t); PrimBXor t -> n "bxor" (int t); PrimBNot t -> n "bnot" (int t)
  PrimBShiftL t -> n "shl" (int t); PrimBShiftR t -> n "shr" (int t); PrimBRotateL t -> n "rotl" (int t); PrimBRotateR t -> n "rotr" (int t)
  PrimPopCount t -> n "popcount" (int t); PrimCountLeadingZeros t -> n "clz" (int t); PrimCountTrailingZeros t -> n "ctz" (int t)
  PrimFDiv t -> n "fdiv" (flt t); PrimRecip t -> n "recip" (flt t)
  PrimSin t -> n "sin" (flt t); PrimCos t -> n "cos" (flt t); PrimTan t -> n "tan" (flt t)
  PrimAsin t -> n "asin" (flt t); PrimAcos t -> n "acos" (flt t); PrimAtan t -> n "atan" (flt t)
  PrimSinh t -> n "sinh" (flt t); PrimCosh t -> n "cosh" (flt t); PrimTanh t -> n "tanh" (flt t)
  PrimAsinh t -> n "asinh" (flt t); PrimAcosh t -> n "acosh" (flt t); PrimAtanh t -> n "atanh" (flt t)
  PrimExpFloating t -> n "exp" (flt t); PrimSqrt t -> n "sqrt" (flt t); PrimLog t -> n "log" (flt t)
  PrimFPow t -> n "fpow" (flt t); PrimLogBase t -> n "logbase" (flt t); PrimAtan2 t -> n "atan2" (flt t)
  PrimTruncate a b -> n2 "truncate" (flt a) (int b); PrimRound a b -> n2 "round" (flt a) (int b)
  PrimFloor a b -> n2 "floor" (flt a) (int b); PrimCeiling a b -> n2 "ceiling" (flt a) (int b)
  PrimIsNaN t -> n "isnan" (flt t); PrimIsInfinite t -> n "isinf" (flt t)
  PrimLt t -> n "lt" (sgl t); PrimGt t -> n "gt" (sgl t); PrimLtEq t -> n "le" (sgl t); PrimGtEq t -> n "ge" (sgl t)
  PrimEq t -> n "eq" (sgl t); PrimNEq t -> n "ne" (sgl t); PrimMax t -> n "max" (sgl t); PrimMin t -> n "min" (sgl t)
  PrimLAnd -> sx ["prim", "land", x]; PrimLOr -> sx ["prim", "lor", x]; PrimLNot -> sx ["prim", "lnot", x]
  PrimFromIntegral a b -> n2 "fromintegral" (int a) (num b); PrimToFloating a b -> n2 "tofloating" (num a) (flt b)
  where
    n  name t     = sx ["prim", name, t, x]
    n2 name t1 t2 = sx ["prim", name, t1, t2, x]
    num :: NumType t -> String
    num = scalarText . SingleScalarType . NumSingleType
    int :: IntegralType t -> String
    int = num . IntegralNumType
    flt :: FloatingType t -> String
    flt = num . FloatingNumType
    sgl :: SingleType t -> String
    sgl = scalarText . SingleScalarType
