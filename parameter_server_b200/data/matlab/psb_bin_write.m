function psb_bin_write(name, A, varargin)
% PSB_BIN_WRITE  Save a matrix as name.{info,offset,index,value} for the data readers (format: BIN).
%   psb_bin_write(name, A)                        row-major, 8-byte indices, float values
%   psb_bin_write(name, A, 'binary', true)        keep only the pattern (no .value file)
%   psb_bin_write(name, A, 'row_major', false)    column-major (what the block solver reads per feature block)
%   psb_bin_write(name, A, 'sizeof_index', 4)     4-byte indices
%   psb_bin_write(name, A, 'label', y)            also writes name.label (float)
% Counterpart of the reference's mat2bin.m (src/data/matlab/mat2bin.m).
  p = inputParser;
  addParameter(p, 'binary', false); addParameter(p, 'row_major', true);
  addParameter(p, 'sizeof_index', 8); addParameter(p, 'label', []);
  parse(p, varargin{:}); o = p.Results;
  [rows, cols] = size(A);
  fid = fopen([name '.info'], 'w');
  if fid < 0, error('psb:io', 'cannot create %s.info', name); end
  closer = onCleanup(@() fclose(fid));
  tf = {'false', 'true'};
  if ~issparse(A)
    fprintf(fid, 'type: DENSE\nrow_major: %s\n', tf{o.row_major + 1});
    fprintf(fid, 'row { begin: 0 end: %d }\ncol { begin: 0 end: %d }\nnnz: %d\nsizeof_index: %d\nsizeof_value: 4\n', ...
            rows, cols, rows * cols, o.sizeof_index);
    if o.row_major, A = A'; end
    psb_array_write([name '.value'], A, 'single');
  else
    if o.row_major, B = A'; else, B = A; end                      % columns of B are the outer dimension
    [inner, ~, val] = find(B);
    off = [0; cumsum(full(sum(B ~= 0, 1)))'];
    kind = 'SPARSE'; if o.binary, kind = 'SPARSE_BINARY'; end
    fprintf(fid, 'type: %s\nrow_major: %s\n', kind, tf{o.row_major + 1});
    fprintf(fid, 'row { begin: 0 end: %d }\ncol { begin: 0 end: %d }\nnnz: %d\nsizeof_index: %d\nsizeof_value: 4\n', ...
            rows, cols, numel(inner), o.sizeof_index);
    psb_array_write([name '.offset'], uint64(off), 'uint64');
    itype = 'uint64'; if o.sizeof_index == 4, itype = 'uint32'; end
    psb_array_write([name '.index'], cast(inner - 1, itype), itype);
    if ~o.binary, psb_array_write([name '.value'], single(val), 'single'); end
  end
  if ~isempty(o.label), psb_array_write([name '.label'], single(o.label), 'single'); end
end
